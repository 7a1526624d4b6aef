"""Host logic of the Euler sampler, no GPU: the sigma schedule against the reference's
known-answer checks (tests/test_h3.c:101-124) and the op sequence of the three guidance modes
against a recording stand-in for the device context."""
import numpy as np
import pytest


@pytest.fixture(scope="module")
def pkg():
    import __graft_entry__ as entry
    return entry.load_package()


def test_serving_sigmas_known_answers(pkg):
    s50 = pkg.serving_sigmas(50)
    assert s50[0] == 1.0 and s50[50] == 0.0
    assert abs(s50[25] - np.float32(12.0 * 0.5 / (1.0 + 11.0 * 0.5))) <= 1e-7
    assert np.all(np.diff(s50) < 0)
    s4 = pkg.serving_sigmas(4)
    assert s4[0] == 1.0 and s4[4] == 0.0
    assert abs(s4[1] - 36.0 / 37.0) <= 1e-7
    a4 = pkg.serving_sigmas(4, shift=3.0)      # the audio stream's shift (h3_host.h:13)
    assert abs(a4[1] - 9.0 / 10.0) <= 1e-7
    assert np.all(np.diff(a4) < 0)


def test_reuse_schedule_known_answers(pkg):
    """tests/test_h3.c:128-147 of the reference."""
    sel = pkg.reuse_schedule(20, 3)
    assert sum(sel) == 8 and [i for i, v in enumerate(sel) if v] == [0, 3, 6, 9, 12, 15, 18, 19]
    sel = pkg.reuse_schedule(20, 2)
    assert sum(sel) == 11 and all(v == (i % 2 == 0 or i == 19) for i, v in enumerate(sel))
    sel = pkg.reuse_schedule(50, 3)
    assert sum(sel) == 18 and all(v == (i % 3 == 0 or i == 49) for i, v in enumerate(sel))
    assert sum(pkg.reuse_schedule(20, 1)) == 20
    with pytest.raises(ValueError):
        pkg.reuse_schedule(20, 33)


def test_extrapolation_ratio(pkg):
    assert pkg.extrapolation_ratio(0.5, 0.6, 0.7, False) == 0.0
    assert abs(pkg.extrapolation_ratio(0.5, 0.6, 0.7, True) - 1.0) < 1e-6      # one interval further
    assert pkg.extrapolation_ratio(0.0, 0.6, 0.7, True) == 2.0                  # clamped
    assert pkg.extrapolation_ratio(0.5, 0.6, 0.6, True) == 0.0                  # degenerate schedule


class FakeTensor:
    def __init__(self, name):
        self.name = name


class FakeGpu:
    def __init__(self):
        self.log = []

    def new(self, n, dtype):
        return FakeTensor(f"new{n}")

    def begin(self):
        self.log.append("begin")

    def submit(self):
        self.log.append("submit")

    def flush(self):
        self.log.append("flush")

    def op(self, name, *args):
        self.log.append((name,) + tuple(a.name if isinstance(a, FakeTensor) else a for a in args))


class FakeStep:
    """Stands in for DenoiseStep: records which text and row maps each forward used."""

    def __init__(self, gpu, pkg):
        class D:
            pass
        self.dit = D()
        self.dit.gpu, self.dit.s = gpu, pkg.DitShape()
        self.video_rows = 10
        self.text_hidden = FakeTensor("cond_text")
        self.velocity = FakeTensor("velocity")
        self.row_map = self.final_row_map = None

    def forward(self):
        self.dit.gpu.log.append(("forward", self.text_hidden.name, self.row_map.name, self.final_row_map.name))

    def euler(self, delta, ratio=0.0, previous=None):
        entry = ("euler", round(delta, 6))
        if ratio or previous is not None:
            entry += (round(ratio, 6), previous.name if previous is not None else None)
        self.dit.gpu.log.append(entry)


def maps(n):
    return [FakeTensor(f"rm{i}") for i in range(n)], [FakeTensor(f"frm{i}") for i in range(n)]


def test_plain_loop(pkg):
    gpu = FakeGpu()
    step = FakeStep(gpu, pkg)
    sig = np.array([1.0, 0.5, 0.0], np.float32)
    pkg.EulerSampler(step, sig, *maps(2)).run()
    assert gpu.log == ["begin", ("forward", "cond_text", "rm0", "frm0"), ("euler", 0.5), "flush",
                       ("forward", "cond_text", "rm1", "frm1"), ("euler", 0.5), "submit"]


def test_reuse_loop(pkg):
    """5 steps, interval 2: steps 0, 2, 4 evaluate; 1 reuses the only velocity, 3 extrapolates."""
    gpu = FakeGpu()
    step = FakeStep(gpu, pkg)
    sig = np.array([1.0, 0.8, 0.6, 0.4, 0.2, 0.0], np.float32)
    pkg.EulerSampler(step, sig, *maps(5), reuse_interval=2).run()
    f = lambda i: ("forward", "cond_text", f"rm{i}", f"frm{i}")
    keep = ("copy_bf16", "new960", 0, "velocity", 0, 960)
    assert gpu.log == ["begin", f(0), ("euler", 0.2), "flush",
                       ("euler", 0.2),
                       keep, f(2), ("euler", 0.2, 0.0, "new960"), "flush",
                       ("euler", 0.2, 0.5, "new960"),
                       keep, f(4), ("euler", 0.2, 0.0, "new960"), "submit"]


def test_sequential_guidance(pkg):
    gpu = FakeGpu()
    step = FakeStep(gpu, pkg)
    sig = np.array([1.0, 0.0], np.float32)
    pkg.EulerSampler(step, sig, *maps(1), guidance=2.5, uncond_text=FakeTensor("uncond_text")).run()
    assert gpu.log == ["begin", ("forward", "cond_text", "rm0", "frm0"),
                       ("copy_bf16", "new960", 0, "velocity", 0, 960),
                       ("forward", "uncond_text", "rm0", "frm0"),
                       ("h3x_cfg_combine_bf16", "velocity", "new960", "velocity", 960, 2.5),
                       ("euler", 1.0), "submit"]
    assert step.text_hidden.name == "cond_text"


@pytest.mark.parametrize("is_cond", [True, False])
def test_paired_guidance(pkg, is_cond):
    gpu = FakeGpu()
    step = FakeStep(gpu, pkg)

    class Pair:
        def swap(self, out, inp):
            gpu.log.append(("swap", out.name, inp.name))
    pair = Pair()
    pair.is_cond = is_cond
    pkg.EulerSampler(step, np.array([1.0, 0.0], np.float32), *maps(1), guidance=4.0, pair=pair).run()
    combine = ("h3x_cfg_combine_bf16", "velocity") + (("velocity", "new960") if is_cond else ("new960", "velocity")) + (960, 4.0)
    assert gpu.log == ["begin", ("forward", "cond_text", "rm0", "frm0"), ("swap", "new960", "velocity"),
                       combine, ("euler", 1.0), "submit"]


def test_guidance_needs_one_source(pkg):
    gpu = FakeGpu()
    with pytest.raises(ValueError):
        pkg.EulerSampler(FakeStep(gpu, pkg), np.array([1.0, 0.0], np.float32), *maps(1), guidance=2.0)


def test_cfg_combine_oracle_formula():
    import h3_oracle as o
    rng = np.random.default_rng(0)
    c = o.to_bf16(rng.standard_normal(1000, dtype=np.float32))
    u = o.to_bf16(rng.standard_normal(1000, dtype=np.float32))
    got = o.from_bf16(o.cfg_combine_bf16(c, u, 3.0))
    cf, uf = o.from_bf16(c).astype(np.float64), o.from_bf16(u).astype(np.float64)
    want = uf + 3.0 * (cf - uf)
    assert np.all(np.abs(got - want) <= np.abs(want) * 2.0 ** -8 + 1e-30)
    assert np.array_equal(o.cfg_combine_bf16(c, u, 1.0), c)     # guidance 1 returns cond exactly


def test_oracle_masked_attention_reduces_to_dense_cases():
    """The CPU oracle's block-sparse attention: a mask listing every tile is the dense result,
    and a block restricted to one 64-key tile equals dense attention over those 64 keys."""
    import h3_oracle as o
    rng = np.random.default_rng(0)
    S, H = 200, 2
    q, k, v = [o.to_bf16(rng.standard_normal(S * H * 128, dtype=np.float32)) for _ in range(3)]
    qb, kt = (S + 127) // 128, (S + 63) // 64
    ptr = np.arange(qb + 1, dtype=np.uint32) * kt
    idx = np.tile(np.arange(kt, dtype=np.uint32), qb)
    dense = o.sdpa_bf16(q, k, v, S, H, 128, 0.088, round_p=1)
    assert np.array_equal(o.sdpa_bf16_sparse(q, k, v, S, H, 128, 0.088, ptr, idx, round_p=1), dense)
    ptr = np.array([0, 1, 1 + kt], np.uint32)
    idx = np.concatenate([[0], np.arange(kt)]).astype(np.uint32)
    got = o.sdpa_bf16_sparse(q, k, v, S, H, 128, 0.088, ptr, idx, round_p=1).reshape(S, H, 128)
    first = [a.reshape(S, H, 128)[:64].reshape(-1) for a in (q, k, v)]
    small = o.sdpa_bf16(*first, 64, H, 128, 0.088, round_p=1).reshape(64, H, 128)
    assert np.array_equal(got[:64], small)
