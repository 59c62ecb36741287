"""splash_b200: B200-native DFlash2 verify-step kernels behind a C ABI (include/splash_b200.h).

The Python in this package is a thin ctypes harness over libsplash_b200.so for tests and the
benchmark; the product is the shared library and its C++ host operator layer."""
