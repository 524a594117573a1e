"""KMeans engine, its drivers and a host estimator.  Importing this package loads
libkmb200.so and fails if it has not been built."""
from . import drivers  # noqa: F401
from ._host import KMeans  # noqa: F401
from .engine import KMeansEngine  # noqa: F401
