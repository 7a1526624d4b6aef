"""The drop-in boundary itself (reference h3_gpu.h / h3_gpu_cuda.cu conventions): command
model, error reporting, statistics, tensor I/O (host ranges, files, streaming), casts and
copies, and the stubs for entry points that are not on the DiT path."""
import ctypes as C

import numpy as np
import pytest

import h3_oracle as o

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def pkg():
    import __graft_entry__ as entry
    return entry.load_package()


@pytest.fixture()
def gpu(pkg):
    g = pkg.Gpu(0)
    yield g
    g.close()


def test_ops_need_an_active_command_and_begin_does_not_nest(gpu, pkg):
    """h3_cuda_internal.h:163-167 (ops fail outside begin..submit), h3_gpu_cuda.cu:871-878."""
    a, b = gpu.bf16(o.normal_bf16(64, 1)), gpu.bf16(o.normal_bf16(64, 2))
    out = gpu.new(64, pkg.BF16)
    assert not gpu.try_op("add_bf16", out, a, b, 64)
    assert "no active command buffer" in gpu.error()
    lib = gpu.lib
    assert lib.h3_gpu_begin(gpu.handle) == 1
    assert lib.h3_gpu_begin(gpu.handle) == 0            # already active
    assert gpu.try_op("add_bf16", out, a, b, 64)
    assert lib.h3_gpu_continue(gpu.handle) == 1         # flush hint keeps the command open
    assert gpu.try_op("sub_bf16", out, a, b, 64)
    assert lib.h3_gpu_submit(gpu.handle) == 1
    assert lib.h3_gpu_submit(gpu.handle) == 0           # nothing active any more
    assert lib.h3_gpu_continue(gpu.handle) == 0
    want = o.sub_bf16(o.normal_bf16(64, 1), o.normal_bf16(64, 2))
    assert np.array_equal(out.read(), want)


def test_validation_errors_are_reported_not_fatal(gpu, pkg):
    a = gpu.bf16(o.normal_bf16(64, 1))
    f = gpu.f32(np.zeros(64, np.float32))
    out = gpu.new(32, pkg.BF16)
    gpu.begin()
    assert not gpu.try_op("add_bf16", out, a, a, 64)          # output too small
    assert "too small" in gpu.error()
    assert not gpu.try_op("add_bf16", a, a, f, 64)            # dtype mismatch
    assert "dtype" in gpu.error()
    assert gpu.try_op("add_bf16", a, a, a, 64)                # the context is still usable
    gpu.submit()
    with pytest.raises(pkg.H3Error):
        gpu.op("add_bf16", out, a, a, 64)                     # outside a command, through the raising form


def test_statistics_follow_the_reference_rules(gpu, pkg):
    """+1 linear dispatch only for rows >= 32, in >= 256, out >= 256 (h3_cuda_core.cu:838-841);
    +2 per MLP; +1 SDPA per attention call; hand kernels count as direct dispatches."""
    rows, k, n = 64, 256, 256
    x, w = gpu.bf16(o.normal_bf16(rows * k, 1)), gpu.bf16(o.normal_bf16(n * k, 2, 0.0, 0.05))
    small_w = gpu.bf16(o.normal_bf16(8 * k, 3, 0.0, 0.05))
    out, small = gpu.new(rows * n, pkg.BF16), gpu.new(rows * 8, pkg.BF16)
    fc1, fc2 = gpu.bf16(o.normal_bf16(2 * 512 * k, 4, 0.0, 0.05)), gpu.bf16(o.normal_bf16(n * 512, 5, 0.0, 0.05))
    q = gpu.bf16(o.normal_bf16(64 * 2 * 128, 6))
    att = gpu.new(64 * 2 * 128, pkg.BF16)
    before = gpu.stats()
    gpu.begin()
    gpu.op("linear_bf16", out, x, w, None, rows, k, n)
    gpu.op("linear_bf16", small, x, small_w, None, rows, k, 8)      # out < 256: a direct dispatch
    gpu.op("mlp_bf16", out, x, fc1, fc2, rows, k, 512, n)
    gpu.op("sdpa_bf16", att, q, q, q, 64, 2, 128, 0.088)
    gpu.op("add_bf16", out, out, out, rows * n)
    gpu.submit()
    after = gpu.stats()
    assert after.mps_linear_dispatches - before.mps_linear_dispatches == 3
    assert after.mps_sdpa_dispatches - before.mps_sdpa_dispatches == 1
    assert after.direct_dispatches - before.direct_dispatches == 2
    assert after.submissions - before.submissions == 1
    assert after.tensor_allocations >= 8 and after.live_bytes > 0 and after.peak_live_bytes >= after.live_bytes


def test_host_ranges_casts_and_copies(gpu, pkg):
    rng = np.random.default_rng(0)
    values = rng.standard_normal(300, dtype=np.float32)
    t = gpu.f32(values)
    lib = gpu.lib
    assert lib.h3_gpu_tensor_elements(t.handle) == 300 and lib.h3_gpu_tensor_dtype(t.handle) == pkg.F32
    part = np.empty(50, np.float32)
    assert lib.h3_gpu_tensor_read_f32_range(t.handle, 100, part.ctypes.data, 50) == 1
    assert np.array_equal(part, values[100:150])
    assert lib.h3_gpu_tensor_read_f32_range(t.handle, 280, part.ctypes.data, 50) == 0      # past the end
    patch = np.arange(10, dtype=np.float32)
    assert lib.h3_gpu_tensor_write_f32_range(t.handle, 5, patch.ctypes.data, 10) == 1
    assert lib.h3_gpu_tensor_write_f32_range(t.handle, 295, patch.ctypes.data, 10) == 0
    values[5:15] = patch
    assert np.array_equal(t.read(), values)
    b, back = gpu.new(300, pkg.BF16), gpu.new(300, pkg.F32)
    dst = gpu.bf16(np.zeros(400, np.uint16))
    gpu.begin()
    gpu.op("cast_f32_to_bf16", b, t, 300)
    gpu.op("cast_bf16_to_f32", back, b, 300)
    gpu.op("copy_bf16", dst, 50, b, 100, 200)
    gpu.submit()
    want = o.to_bf16(values)
    assert np.array_equal(b.read(), want)
    assert np.array_equal(back.read(), o.from_bf16(want))
    got = dst.read()
    assert np.array_equal(got[50:250], want[100:300]) and not got[:50].any() and not got[250:].any()
    piece = o.normal_bf16(20, 9)
    assert lib.h3_gpu_tensor_write_bf16_range(dst.handle, 380, piece.ctypes.data, 20) == 1
    assert lib.h3_gpu_tensor_write_bf16_range(dst.handle, 390, piece.ctypes.data, 20) == 0
    assert np.array_equal(dst.read()[380:], piece)


def test_file_loads_and_streaming(gpu, pkg, tmp_path):
    """tensor_load_* / tensor_read_file_bf16 / tensor_stream_file_bf16 (h3_gpu_cuda.cu:426-776):
    payloads at a byte offset inside a larger file, short files are errors."""
    rng = np.random.default_rng(1)
    bf16 = o.to_bf16(rng.standard_normal(5000, dtype=np.float32))
    f32 = rng.standard_normal(700, dtype=np.float32)
    path = tmp_path / "weights.bin"
    header = b"x" * 24
    path.write_bytes(header + bf16.tobytes() + f32.tobytes())
    lib, p = gpu.lib, str(path).encode()
    h = lib.h3_gpu_tensor_load_bf16(gpu.handle, p, 24, 5000)
    assert h
    loaded = pkg.Tensor(gpu, h, 5000, pkg.BF16)
    assert np.array_equal(loaded.read(), bf16)
    h = lib.h3_gpu_tensor_load_f32(gpu.handle, p, 24 + 10000, 700)
    assert h and np.array_equal(pkg.Tensor(gpu, h, 700, pkg.F32).read(), f32)
    assert not lib.h3_gpu_tensor_load_bf16(gpu.handle, p, 24 + 10000, 5000)       # runs past the end of the file
    assert not lib.h3_gpu_tensor_load_bf16(gpu.handle, str(tmp_path / "missing.bin").encode(), 0, 16)
    target = gpu.new(5000, pkg.BF16)
    err = C.create_string_buffer(256)
    assert lib.h3_gpu_tensor_read_file_bf16(target.handle, p, 24 + 2 * 1000, 3000, err, 256) == 1
    assert np.array_equal(target.read(3000), bf16[1000:4000])
    assert lib.h3_gpu_tensor_stream_file_bf16(target.handle, p, 24, 5000, err, 256) == 1
    gpu.begin(); gpu.submit()                                 # a command boundary orders the streamed copy
    assert np.array_equal(target.read(), bf16)
    assert lib.h3_gpu_tensor_read_file_bf16(target.handle, p, 24, 6000, err, 256) == 0   # larger than the tensor
    assert err.value


@pytest.mark.parametrize("direct", ["1", "0"])
def test_large_file_loads_cross_chunk_boundaries(pkg, tmp_path, monkeypatch, direct):
    """A payload of several 16 MiB chunks at an odd byte offset: the chunked, multi-threaded
    reader (with and without O_DIRECT) must deliver every byte in place, also when the ring of
    staging buffers wraps (more chunks than buffers) and when the tensor is filled twice."""
    monkeypatch.setenv("H3B_DIRECT_IO", direct)
    rng = np.random.default_rng(3)
    elements = (120 << 20) // 2 + 12345                     # ~120 MiB of BF16: 8 chunks > 6 buffers
    payload = rng.integers(0, 1 << 16, elements, dtype=np.uint16)
    path = tmp_path / "big.bin"
    with open(path, "wb") as f:
        f.write(b"h" * 4099)                                # payload starts off the 4 KiB grid
        f.write(payload.tobytes())
        f.write(b"t" * 100)
    g = pkg.Gpu(0)
    try:
        lib, p = g.lib, str(path).encode()
        h = lib.h3_gpu_tensor_load_bf16(g.handle, p, 4099, elements)
        assert h, g.error()
        t = pkg.Tensor(g, h, elements, pkg.BF16)
        assert np.array_equal(t.read(), payload)
        err = C.create_string_buffer(256)
        # a window in the middle, into the same tensor, through the streaming entry point
        assert lib.h3_gpu_tensor_stream_file_bf16(t.handle, p, 4099 + 2 * 1000001, 20_000_000, err, 256) == 1
        assert np.array_equal(t.read(20_000_000), payload[1000001:21000001])
        assert lib.h3_gpu_tensor_read_file_bf16(t.handle, p, 4099, elements + 100, err, 256) == 0
    finally:
        g.close()


def test_op_profile_prints_device_time_per_op(pkg, monkeypatch, capfd):
    """H3_PROFILE=2: h3_gpu_profile_mark prints, per op name, the device time measured with
    events on the context's stream (the reference prints wall/wait per phase only,
    h3_gpu_cuda.cu:21-45,919-933)."""
    monkeypatch.setenv("H3_PROFILE", "2")
    g = pkg.Gpu(0)
    try:
        a = g.bf16(o.normal_bf16(1 << 16, 1))
        out = g.new(1 << 16, pkg.BF16)
        g.begin()
        for _ in range(3):
            g.op("add_bf16", out, a, a, 1 << 16)
        g.op("silu_bf16", out, a, 1 << 16)
        g.submit()
        g.lib.h3_gpu_profile_set_label(g.handle, b"probe")
        g.lib.h3_gpu_profile_mark(g.handle, b"elementwise")
    finally:
        g.close()
    err = capfd.readouterr().err
    assert "[probe] elementwise" in err
    rows = [line for line in err.splitlines() if "launches" in line]
    assert any("add_bf16" in r and " 3 launches" in r for r in rows), err
    assert any("silu_bf16" in r and " 1 launches" in r for r in rows), err


def test_entry_points_off_the_dit_path_fail_with_a_message(gpu, pkg):
    """The reference's practice for unported ops: return 0 and say so (h3_cuda_dit.cu:1072-1216)."""
    lib = gpu.lib
    gpu.begin()
    fn = lib.h3_gpu_conv3d_f32
    fn.restype = C.c_int
    fn.argtypes = None
    assert fn(C.c_void_p(gpu.handle)) == 0        # the stub reads only the context argument
    assert "not" in gpu.error().lower()
    gpu.submit()
    assert lib.h3_gpu_is_m5(gpu.handle) == 0 and lib.h3_gpu_has_int8_mlp(gpu.handle) == 0
    assert lib.h3_gpu_prefers_gpu_sampler(gpu.handle) == 1


def test_cuda_probe_fills_the_reference_struct(gpu, pkg):
    """h3_cuda_probe (h3_cuda.h:9, h3_gpu_cuda.cu:47-79) with the h3_device_info layout of
    h3.h:132-146: name, "sm_XY", host RAM, device memory twice, zeros for the Apple-only fields."""
    class DeviceInfo(C.Structure):
        _fields_ = [("name", C.c_char * 128), ("architecture", C.c_char * 128),
                    ("physical_memory", C.c_uint64), ("recommended_working_set", C.c_uint64),
                    ("max_buffer_length", C.c_uint64), ("apple_gpu_family", C.c_int),
                    ("metal4", C.c_int), ("unified_memory", C.c_int)]
    info, err = DeviceInfo(), C.create_string_buffer(256)
    fn = gpu.lib.h3_cuda_probe
    fn.restype, fn.argtypes = C.c_int, [C.POINTER(DeviceInfo), C.c_char_p, C.c_size_t]
    assert fn(C.byref(info), err, 256) == 1
    assert info.name and info.architecture == b"sm_100"
    assert info.recommended_working_set == info.max_buffer_length > (100 << 30)
    assert info.physical_memory > (1 << 30)
    assert (info.apple_gpu_family, info.metal4, info.unified_memory) == (0, 0, 0)
    assert fn(None, err, 256) == 0


def test_a_bounded_wait_that_runs_out_fails_the_submit_and_leaves_the_context_usable(gpu, pkg):
    """The cross-rank barrier with a peer that never arrives: a two-rank table whose flag words
    are both local buffers, nobody plays rank 1, and a budget of a few milliseconds. The kernel
    returns by itself, h3_gpu_submit reports "peer barrier gave up", the status word is cleared
    and the next command runs. Nothing faults, hangs or is killed."""
    lib = gpu.lib
    flags = [gpu.f32(np.zeros(16, np.float32)) for _ in range(2)]     # 16 zeroed 32-bit words each
    peers = pkg.UlyssesPeers()
    peers.world, peers.rank, peers.rows_local = 2, 0, 1
    for r in range(2):
        peers.flags[r] = flags[r].pointer
    assert lib.h3x_set_wait_budget_cycles(gpu.handle, 0, 4_000_000) == 1      # ~2 ms of SM clock
    gpu.begin()
    assert lib.h3x_set_wait_budget_cycles(gpu.handle, 0, 1) == 0              # not inside a command
    gpu.op("h3x_peer_barrier", peers)
    assert lib.h3_gpu_submit(gpu.handle) == 0
    assert "peer barrier gave up" in gpu.error()
    assert lib.h3x_kernel_status(gpu.handle) == 0                             # cleared by the failed submit
    a = gpu.bf16(o.normal_bf16(64, 1))
    out = gpu.new(64, pkg.BF16)
    gpu.begin()
    gpu.op("add_bf16", out, a, a, 64)
    gpu.submit()                                                              # the context still works
    assert np.array_equal(out.read(), o.add_bf16(o.normal_bf16(64, 1), o.normal_bf16(64, 1)))
    # the same barrier passes once the peer's word is there: rank 1 "arrives" by a host write of
    # the next epoch (2) into this rank's slot for it
    flags[0].write(np.array([2], np.uint32).view(np.float32), offset=1)
    gpu.begin()
    gpu.op("h3x_peer_barrier", peers)
    gpu.submit()
