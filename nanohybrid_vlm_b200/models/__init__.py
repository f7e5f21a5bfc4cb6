"""Built-in architectures.  Importing this package registers them."""
from . import beputar, ginodra, muvonex, nomudra, qwen3  # noqa: F401
