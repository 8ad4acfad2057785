"""B200-native backend for the lanternl language-model token loop.

The package holds the CUDA kernels and C ABI (csrc/, built into luaTL.so), a host-side
mirror of the reference's backend adapter and GPU model (luatl_adapter, gpu_transformer),
and seeded synthetic inputs (synth).  Nothing here computes on the CPU: every model or
operator call goes through luaTL.so and raises if the library or a GPU is missing.
"""
__version__ = "0.1.0"
