"""Built-in architectures: importing this package registers them."""
from . import gemma, pesanex, taritar, zafilix  # noqa: F401
