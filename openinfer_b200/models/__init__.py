"""Built-in architectures. Importing this package registers them."""
from . import delunex, pilonex, qwen3  # noqa: F401
