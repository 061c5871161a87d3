from . import dabodra, llama, mokatar, nibelorn, vitinex  # noqa: F401  (registers the architectures)
