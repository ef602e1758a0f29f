"""Architectures: each module maps its config.json to a ``ModelSpec`` and registers itself by name."""
from . import nanbeige      # noqa: F401
from . import vozinex       # noqa: F401
from . import nilatar       # noqa: F401
from . import medodra       # noqa: F401
from . import luzerax       # noqa: F401
