"""Built-in architectures; importing this package registers them."""
from . import derupel, fonuvik, nasozen, qwen3, sarulix  # noqa: F401
