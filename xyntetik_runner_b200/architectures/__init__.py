"""Architectures this engine knows; importing the package registers them."""
from . import besolix  # noqa: F401
from . import buzarax  # noqa: F401
from . import llama  # noqa: F401
from . import pitolix  # noqa: F401
from . import turudra  # noqa: F401
