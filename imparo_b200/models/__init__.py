"""Built-in architectures; importing this package registers them."""
from . import lfm2  # noqa: F401
from . import vipotar  # noqa: F401
from . import negotar  # noqa: F401
from . import keralix  # noqa: F401
from . import zepesun  # noqa: F401
