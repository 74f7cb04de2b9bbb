"""Built-in architectures. Importing this package registers them."""
from . import delunex, qwen3  # noqa: F401
