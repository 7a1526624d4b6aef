"""h3.c_b200 — B200-native backend for the MiniMax-H3 DiT denoiser forward.

csrc/       CUDA kernels and the C ABI (libh3b200.so, declared in include/h3b200.h)
binding.py  ctypes view of that ABI
peers.py    peer-mapped exchange buffers for the fused sequence-parallel path
dit.py      host-side driver mirroring the reference's run_block / encode_forward
build.py    nvcc build of the shared library (sm_100a)

The directory name contains a dot, so import it through `__graft_entry__.load_package()`
(or importlib with an explicit module name such as `h3c_b200`).
"""
from .binding import (BF16, F32, I8, U32, Gpu, H3Error, Tensor, UlyssesPeers,  # noqa: F401
                      declared_functions, library)
from .peers import PeerExchange  # noqa: F401
from .dit import (BlockWeights, DenoiseStep, Dit, DitShape, EulerSampler, TokenReduction, extrapolation_ratio,
                  reuse_schedule,
                  serving_sigmas, block_tensor_shapes,  # noqa: F401
                  default_inv_freq, grid_positions, row_map_for, shard_rows,
                  ulysses_pack_order)
