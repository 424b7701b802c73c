"""Parsers for the raw files of three small public datasets; none of them downloads anything
(flodl/src/data/datasets/{mnist,cifar10,shakespeare}.rs)."""
from .cifar10 import Cifar10  # noqa: F401
from .mnist import Mnist  # noqa: F401
from .shakespeare import Shakespeare  # noqa: F401
