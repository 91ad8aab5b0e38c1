"""CUDA kernels: building (``build``), loading (``lib``) and calling (``kernels``)."""
