"""attention_b200: B200 (sm_100a) FlashAttention forward and PagedAttention decode.

The product is the native library attention_b200/lib/libahpc_b200.so (C ABI: include/ahpc.h;
C++ surface: include/attention_hpc/).  The Python modules here are the harness around it:

  build   in-tree nvcc build of the library
  abi     ctypes bindings of the C ABI
  ops     torch-tensor front end used by tests and the benchmark
  synth   seeded synthetic workloads (shapes and value distributions of the benchmark configurations)
"""
__version__ = "0.1.0"
