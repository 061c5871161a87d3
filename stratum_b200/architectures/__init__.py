from . import dabodra, llama, nibelorn, vitinex  # noqa: F401  (registers the architectures)
