"""Architectures.  Importing this package registers the built-in ones."""
from . import dumizen, gepadra, phimoe, puledra, tefovik  # noqa: F401
