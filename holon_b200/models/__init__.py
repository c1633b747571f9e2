"""Built-in architectures; importing this package registers them."""
from . import kasovik, qwen3, rulorax, tilarax, vobosun  # noqa: F401
