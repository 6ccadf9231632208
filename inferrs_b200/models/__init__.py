"""Architectures.  Importing the package registers them by the name config.json uses."""
from . import qwen3  # noqa: F401
from . import vebonex  # noqa: F401
from . import tikizen  # noqa: F401
from . import sefalorn  # noqa: F401
from . import ruzunex  # noqa: F401
