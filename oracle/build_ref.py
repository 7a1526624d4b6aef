#!/usr/bin/env python3
"""Build the oracle and, when the reference tree is present, the reference-derived checkers.

TEST INFRASTRUCTURE ONLY. Nothing built here is loaded by the shipped library.

Outputs
-------
oracle/libh3oracle.so          the plain-C restatement (h3_oracle.c); always built.
oracle/_ref/libh3refcpu.so     the reference's own CPU test references (the static
                               ref_* functions of tests/test_cuda_{dit,attention,core}.c)
                               and its host helpers (h3_host.c), compiled from the
                               reference tree where it lies, with tiny exported
                               wrappers (ref_shim_*.c).  Used to pin the restatement.
oracle/_ref/libh3ref.so        the reference's CUDA backend (h3_gpu_cuda.cu + h3_cuda_*.cu)
                               compiled for sm_100: the "reference BF16 path" that the
                               parity bars are stated against; runs only where a GPU is.
oracle/_ref/test_cuda_dit_b200 the reference's own test program tests/test_cuda_dit.c,
                               linked against the B200 library instead of its backend.
oracle/_ref/dit_host_b200      the reference's unmodified DiT host code (loader, schedule, text
oracle/_ref/vae_host_b200      the reference's unmodified video-VAE decoder host + tests/vae_host_driver.c,
oracle/_ref/vae_host_ref       linked against this library / against libh3ref.so
oracle/_ref/dit_host_ref       refiner, run_block, samplers) + tests/dit_host_driver.c, linked
                               against the B200 library / against the reference's CUDA backend.

No reference source is copied: the compiler reads the files in place and only
objects/binaries land under oracle/_ref/ (git-ignored).
"""
from __future__ import annotations

import os
import re
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
REPO = HERE.parent
# the reference tree: H3_REFERENCE_DIR, else a directory named "reference" beside the repository
REF = Path(os.environ.get("H3_REFERENCE_DIR", REPO.parent / "reference"))
OUT = HERE / "_ref"
CUDA_HOME = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))

CPU_FLAGS = ["-O3", "-mavx2", "-mfma", "-ffp-contract=off", "-fopenmp", "-fPIC"]


def run(cmd, **kw):
    print("+", " ".join(str(c) for c in cmd), flush=True)
    subprocess.run([str(c) for c in cmd], check=True, **kw)


def newer(target: Path, sources) -> bool:
    if not target.exists():
        return False
    stamp = target.stat().st_mtime
    return all(Path(s).stat().st_mtime <= stamp for s in sources)


def build_oracle() -> Path:
    target = HERE / "libh3oracle.so"
    sources = [HERE / "h3_oracle.c", HERE / "h3_oracle.h"]
    if not newer(target, sources):
        run(["gcc", "-std=gnu11", *CPU_FLAGS, "-shared", "-o", target,
             HERE / "h3_oracle.c", "-lm"])
    return target


def reference_symbols() -> list[str]:
    """Every h3_gpu_* / h3_cuda_* function the reference's device API declares."""
    text = (REF / "h3_gpu.h").read_text() + (REF / "h3_cuda.h").read_text()
    names = sorted(set(re.findall(r"\b(h3_gpu_[a-z0-9_]+|h3_cuda_probe)\s*\(", text)))
    return names


def build_ref_cpu() -> Path | None:
    """The reference's CPU references, callable: pins h3_oracle.c."""
    if not REF.is_dir():
        return None
    OUT.mkdir(exist_ok=True)
    target = OUT / "libh3refcpu.so"
    shims = [HERE / "ref_shim_dit.c", HERE / "ref_shim_attention.c",
             HERE / "ref_shim_core.c"]
    ref_sources = [REF / "tests/test_cuda_dit.c", REF / "tests/test_cuda_attention.c",
                   REF / "tests/test_cuda_core.c", REF / "h3_host.c"]
    if newer(target, shims + ref_sources + [Path(__file__)]):
        return target
    # The test programs call the device API; they are never run here, so the
    # API is satisfied by inert definitions generated from the header's names.
    stubs = OUT / "device_api_stubs.c"
    stubs.write_text(
        "/* generated: inert device API so the test files' CPU references link */\n"
        + "".join(f"int {n}(void) {{ return 0; }}\n" for n in reference_symbols()))
    objects = []
    for shim in shims:
        obj = OUT / (shim.stem + ".o")
        run(["gcc", "-std=gnu11", *CPU_FLAGS, "-w", "-I", REF, "-I", REF / "tests", "-c", shim,
             "-o", obj])
        objects.append(obj)
    host_obj = OUT / "h3_host.o"
    run(["gcc", "-std=c11", "-D_DEFAULT_SOURCE", *CPU_FLAGS, "-w", "-I", REF, "-c",
         REF / "h3_host.c", "-o", host_obj])
    stub_obj = OUT / "device_api_stubs.o"
    run(["gcc", "-O1", "-fPIC", "-w", "-c", stubs, "-o", stub_obj])
    run(["gcc", "-shared", "-fopenmp", "-o", target, *objects, host_obj, stub_obj, "-lm"])
    return target


def build_ref_cuda() -> Path | None:
    """The reference's own CUDA backend as a separate library (GPU oracle)."""
    if not REF.is_dir() or shutil.which("nvcc") is None:
        return None
    OUT.mkdir(exist_ok=True)
    target = OUT / "libh3ref.so"
    units = ["h3_gpu_cuda.cu", "h3_cuda_gemm.cu", "h3_cuda_core.cu", "h3_cuda_dit.cu",
             "h3_cuda_attention.cu", "h3_cuda_conv.cu"]
    sources = [REF / u for u in units]
    if newer(target, sources + [Path(__file__)]):
        return target
    objects = []
    for unit in units:
        obj = OUT / (Path(unit).stem + ".o")
        if not newer(obj, [REF / unit]):
            run(["nvcc", "-O3", "-std=c++14", "-arch=sm_100", "-DH3_BACKEND_CUDA",
                 "-Xcompiler", "-fPIC", "-w", "-I", REF, "-c", REF / unit, "-o", obj])
        objects.append(obj)
    run(["nvcc", "-shared", "-arch=sm_100", "-o", target, *objects,
         "-L", CUDA_HOME / "lib64", "-lcublasLt", "-lcublas", "-lcudart"])
    return target


def build_ref_tests(product_lib: Path) -> list[Path]:
    """The reference's own op test program, linked against the B200 library."""
    if not REF.is_dir() or not product_lib.exists():
        return []
    OUT.mkdir(exist_ok=True)
    built = []
    for name in ["test_cuda_dit"]:
        target = OUT / f"{name}_b200"
        src = REF / "tests" / f"{name}.c"
        if not newer(target, [src, product_lib]):
            run(["gcc", "-std=c11", "-D_DEFAULT_SOURCE", "-O2", "-w", "-I", REF, src,
                 "-o", target, "-L", product_lib.parent, "-lh3b200",
                 "-Wl,-rpath,$ORIGIN/../../h3.c_b200", "-lm"])
        built.append(target)
    return built


def build_ref_hosts(product_lib: Path) -> list[Path]:
    """The reference's own DiT host (h3_dit.c, h3_dit_schedule.c, h3_host.c, h3_weights.c,
    h3_safetensors.c: loader, text refiner, adaLN schedule, rope and row maps, run_block,
    samplers), compiled unmodified from the reference tree, plus the small driver
    tests/dit_host_driver.c, linked once against the B200 library and once against the
    reference's CUDA backend: the same host code on both backends."""
    if not REF.is_dir() or not product_lib.exists():
        return []
    OUT.mkdir(exist_ok=True)
    units = ["h3_dit.c", "h3_dit_schedule.c", "h3_host.c", "h3_weights.c", "h3_safetensors.c"]
    driver = REPO / "tests" / "dit_host_driver.c"
    objects = []
    for unit in units:
        obj = OUT / ("host_" + Path(unit).stem + ".o")
        if not newer(obj, [REF / unit]):
            run(["gcc", "-std=c11", "-D_DEFAULT_SOURCE", "-DH3_BACKEND_CUDA", "-O2", "-w", "-I", REF,
                 "-c", REF / unit, "-o", obj])
        objects.append(obj)
    driver_obj = OUT / "dit_host_driver.o"
    if not newer(driver_obj, [driver]):
        run(["gcc", "-std=c11", "-D_DEFAULT_SOURCE", "-O2", "-Wall", "-I", REF, "-c", driver, "-o", driver_obj])
    built = []
    target = OUT / "dit_host_b200"
    if not newer(target, [*objects, driver_obj, product_lib]):
        run(["gcc", "-o", target, driver_obj, *objects, "-L", product_lib.parent, "-lh3b200",
             "-Wl,-rpath,$ORIGIN/../../h3.c_b200", "-lpthread", "-lm"])
    built.append(target)
    ref_lib = OUT / "libh3ref.so"
    if ref_lib.exists():
        target = OUT / "dit_host_ref"
        if not newer(target, [*objects, driver_obj, ref_lib]):
            run(["gcc", "-o", target, driver_obj, *objects, "-L", OUT, "-lh3ref",
                 "-Wl,--allow-shlib-undefined", "-Wl,-rpath,$ORIGIN",
                 f"-Wl,-rpath,{CUDA_HOME / 'lib64'}", "-lpthread", "-lm"])
        built.append(target)
    return built


def build_ref_vae_hosts(product_lib: Path) -> list[Path]:
    """The reference's own video-VAE decoder host (h3_video_vae.c with h3_weights.c and
    h3_safetensors.c: loader, latent normalisation, RoPE, the 36-block decoder, tiling, temporal
    chunks and blending), compiled unmodified from the reference tree, plus the small driver
    tests/vae_host_driver.c, linked once against the B200 library and once against the
    reference's CUDA backend."""
    if not REF.is_dir() or not product_lib.exists():
        return []
    OUT.mkdir(exist_ok=True)
    units = ["h3_video_vae.c", "h3_weights.c", "h3_safetensors.c"]
    driver = REPO / "tests" / "vae_host_driver.c"
    objects = []
    for unit in units:
        obj = OUT / ("host_" + Path(unit).stem + ".o")
        if not newer(obj, [REF / unit]):
            run(["gcc", "-std=c11", "-D_DEFAULT_SOURCE", "-DH3_BACKEND_CUDA", "-O2", "-w", "-I", REF,
                 "-c", REF / unit, "-o", obj])
        objects.append(obj)
    driver_obj = OUT / "vae_host_driver.o"
    if not newer(driver_obj, [driver]):
        run(["gcc", "-std=c11", "-D_DEFAULT_SOURCE", "-O2", "-Wall", "-I", REF, "-c", driver, "-o", driver_obj])
    built = []
    target = OUT / "vae_host_b200"
    if not newer(target, [*objects, driver_obj, product_lib]):
        run(["gcc", "-o", target, driver_obj, *objects, "-L", product_lib.parent, "-lh3b200",
             "-Wl,-rpath,$ORIGIN/../../h3.c_b200", "-lpthread", "-lm"])
    built.append(target)
    ref_lib = OUT / "libh3ref.so"
    if ref_lib.exists():
        target = OUT / "vae_host_ref"
        if not newer(target, [*objects, driver_obj, ref_lib]):
            run(["gcc", "-o", target, driver_obj, *objects, "-L", OUT, "-lh3ref",
                 "-Wl,--allow-shlib-undefined", "-Wl,-rpath,$ORIGIN",
                 f"-Wl,-rpath,{CUDA_HOME / 'lib64'}", "-lpthread", "-lm"])
        built.append(target)
    return built


def main() -> int:
    build_oracle()
    build_ref_cpu()
    if "--no-cuda" not in sys.argv:
        build_ref_cuda()
    build_ref_tests(REPO / "h3.c_b200" / "libh3b200.so")
    build_ref_hosts(REPO / "h3.c_b200" / "libh3b200.so")
    build_ref_vae_hosts(REPO / "h3.c_b200" / "libh3b200.so")
    return 0


if __name__ == "__main__":
    sys.exit(main())
