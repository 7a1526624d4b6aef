"""h3x_adaln_linear_bf16_noalloc: the final head for callers that must not allocate.

Some hosts hand all device memory to their own pool before the denoiser runs, or call from a
thread where a driver allocation is not allowed; for them the library offers a final-head
entry point whose scratch is a fixed array inside the library image. This test calls it
through the C ABI twice in a row (with different inputs, so anything left in the shared
scratch by the first call would show) and requires the results to equal those of the
ordinary entry point, h3_gpu_adaln_linear_bf16, bit for bit. The calls include one that fills
the built-in scratch to its last element and one whose width is not a multiple of 8 (the
projection then takes the scalar route). Around every call of the new entry point the free
device memory and the context's allocation counters must not move, and a call beyond the
built-in limit must be rejected with a message rather than run.

Collected last on purpose (file name), so that a run stopping at the first failure has
already run every other test. It creates its own context and passes on its own as well as
after the rest of the suite.
"""
import numpy as np
import pytest

import h3_oracle as o
from parity import assert_aggregate_close

pytestmark = pytest.mark.gpu


def final_head_inputs(seed, rows, width, out_dim, slots, offset):
    x = o.normal_bf16(rows * width + offset, seed, 0.0, 2.0)
    norm = o.normal_bf16(width, seed + 1, 0.0, 1.0)
    mod = o.normal_bf16(3 * slots * width, seed + 2, 0.0, 0.5)
    w = o.normal_bf16(out_dim * width, seed + 3, 0.0, 0.02)
    b = o.normal_bf16(out_dim, seed + 4, 0.0, 0.1)
    row_map = (np.arange(rows, dtype=np.uint32) % 3).astype(np.uint32)
    return x, norm, mod, w, b, row_map


def test_no_alloc_final_head_matches_the_allocating_entry_point():
    import __graft_entry__ as entry
    pkg = entry.load_package()
    import torch
    torch.cuda.init()
    gpu = pkg.Gpu(0)
    try:
        slots = 2
        # calls in a row; the second is smaller and offset so stale scratch would matter, the
        # third uses every element of the 4 Mi scratch, the fourth has an odd width
        for seed, rows, width, out_dim, offset in ((11, 96, 5376, 96, 0), (23, 40, 2048, 32, 2048),
                                                   (31, 2048, 2048, 32, 0), (37, 10, 1001, 9, 3)):
            x, norm, mod, w, b, row_map = final_head_inputs(seed, rows, width, out_dim, slots, offset)
            tx, tn, tm, tw, tb = (gpu.bf16(a) for a in (x, norm, mod, w, b))
            tr = gpu.u32(row_map)
            results = {}
            for name in ("h3_gpu_adaln_linear_bf16", "h3x_adaln_linear_bf16_noalloc"):
                out = gpu.bf16(np.zeros(rows * out_dim, np.uint16))
                inv = gpu.f32(np.zeros(rows, np.float32))
                torch.cuda.synchronize()
                free_before, counters_before = torch.cuda.mem_get_info(0)[0], gpu.stats()
                gpu.begin()
                gpu.op(name, out, inv, tx, offset, tn, tm, tr, tw, tb, rows, width, out_dim, slots,
                       0, 1, 1e-5)
                gpu.submit()
                if name.endswith("noalloc"):
                    # the allocating entry point ran the same kernels just before, so nothing is
                    # loaded lazily here: any change would be an allocation
                    counters = gpu.stats()
                    assert torch.cuda.mem_get_info(0)[0] == free_before, "device memory was allocated"
                    assert counters.tensor_allocations == counters_before.tensor_allocations
                    assert counters.allocated_bytes == counters_before.allocated_bytes
                results[name] = (out.read(), inv.read())
            want, got = results["h3_gpu_adaln_linear_bf16"], results["h3x_adaln_linear_bf16_noalloc"]
            assert np.array_equal(got[0], want[0]), f"output differs (rows={rows}, width={width})"
            assert np.array_equal(got[1].view(np.uint32), want[1].view(np.uint32))
            ref_out, _ = o.adaln_linear_bf16(x[offset:], norm, mod, row_map, w, b, rows, width, out_dim,
                                             slots, 0, 1)
            # and both agree with the CPU oracle (composite op: aggregate bound)
            assert_aggregate_close(got[0], ref_out, "no-alloc final head vs oracle")
        # beyond the built-in scratch: rejected, nothing launched
        rows, width = 1024, 5376                       # 5.5 Mi elements > 4 Mi
        big = gpu.new(rows * width, pkg.BF16)
        out, inv = gpu.new(rows * 96, pkg.BF16), gpu.new(rows, pkg.F32)
        gpu.begin()
        before = gpu.stats()
        ok = gpu.try_op("h3x_adaln_linear_bf16_noalloc", out, inv, big, 0, tn, tm, tr, tw, tb, rows,
                        width, 96, slots, 0, 1, 1e-5)
        after = gpu.stats()
        gpu.submit()
        assert not ok and "exceeds the built-in scratch" in gpu.error()
        assert after.direct_dispatches == before.direct_dispatches
        assert after.mps_linear_dispatches == before.mps_linear_dispatches
    finally:
        gpu.close()
