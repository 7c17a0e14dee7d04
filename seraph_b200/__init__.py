"""seraph_b200: B200-native training backward path behind Seraph's C training API.

The product is `libseraph_b200.so` (sources in `csrc/`, C ABI in `include/`);
`seraph_b200.api` is a ctypes mirror of that ABI used by the tests and the
benchmark, `seraph_b200.build` compiles the library in-tree."""
from .api import LIB_PATH  # noqa: F401
