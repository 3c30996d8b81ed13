"""Architecture builders.  Importing this package registers them."""
from . import bavutar, minimax_m2  # noqa: F401
