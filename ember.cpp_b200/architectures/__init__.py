"""Architectures: each module turns its configuration into a ModelSpec and registers itself."""
from . import gpt2, muzozen, nipolorn, sosutar, vipolix  # noqa: F401
