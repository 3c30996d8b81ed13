"""Architecture builders.  Importing this package registers them."""
from . import bavutar, minimax_m2, zisevik  # noqa: F401
