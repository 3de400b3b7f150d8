"""Built-in architectures; importing this package registers them."""

from . import kapitar, llama, pufevik, venezen, vizotar  # noqa: F401
