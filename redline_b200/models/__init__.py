"""Built-in architectures; importing this package registers them."""

from . import kapitar, llama, pufevik, vizotar  # noqa: F401
