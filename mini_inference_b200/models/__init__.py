"""Built-in architectures; importing this package registers them."""
from . import naditar, namesun, qwen3  # noqa: F401
