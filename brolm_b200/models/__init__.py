"""Architectures this framework knows.  Importing the package registers them."""
from . import banevik, gemma2, kedasun, neburax, ritirax  # noqa: F401
