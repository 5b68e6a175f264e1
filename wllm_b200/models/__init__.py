"""Built-in architectures: importing this package registers them."""
from . import gemma  # noqa: F401
