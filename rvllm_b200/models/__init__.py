"""Architectures.  Importing the package registers them; another architecture is one
more module here: a typed configuration, a function from it to a `ModelSpec`, and a
`register_architecture` call."""
from . import bizenex, lfm2, mevuvik, retorax, vifanex  # noqa: F401
