"""Built-in architectures; importing this package registers them."""
from . import naditar, qwen3  # noqa: F401
