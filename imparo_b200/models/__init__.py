"""Built-in architectures; importing this package registers them."""
from . import lfm2  # noqa: F401
