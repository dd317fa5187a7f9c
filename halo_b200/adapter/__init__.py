"""C++23 adapter: halo::backend::Backend over libhalo_cuda.so (cuda_backend.h / cuda_backend.cpp)."""
