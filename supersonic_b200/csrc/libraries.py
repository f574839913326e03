"""Importing this module registers every kernel library of the package with the builder,
so that ``build_all`` compiles all of them."""
from . import build  # noqa: F401

# plain_ops and sampling are registered by build.py itself; faster libraries add themselves here.
