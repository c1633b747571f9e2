"""Built-in architectures; importing this package registers them."""
from . import kasovik, qwen3, rulorax, tilarax  # noqa: F401
