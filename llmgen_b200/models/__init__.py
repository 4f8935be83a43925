"""Built-in architectures; importing this package registers them."""
from . import derupel, fonuvik, qwen3, sarulix  # noqa: F401
