"""Built-in architectures: importing this package registers them."""
from . import gemma, gudarax, pesanex, taritar, zafilix  # noqa: F401
