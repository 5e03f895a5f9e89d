"""tiny_dpcpp_nn for NVIDIA B200: same public names as the reference package
(dpcpp_bindings/tiny_dpcpp_nn/__init__.py:1-8)."""
from .modules import Network, Encoding, NetworkWithInputEncoding, free_temporary_memory  # noqa: F401
