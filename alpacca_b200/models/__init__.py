"""The built-in architectures; importing this package registers them."""
from . import llama  # noqa: F401
