"""Built-in architectures; importing this package registers them."""
from . import llama, rupotar, vonulorn  # noqa: F401
