"""Native libraries of the decode hot path: csrc/<name>.cu built by nvcc for sm_100a on first use, cached in-tree
under _native/ keyed by the command and every source byte, and loaded with ctypes. pointer() and stream() are the
kernels' ctypes arguments.

Same mechanism and names as the reference's loader (native.py:27-65: native_library, cuda_library, pointer,
stream), with the Blackwell arch-specific target instead of sm_90a. There is no fallback: a missing compiler or a
failed build raises, and so does a non-zero status from any entry point (check())."""

import ctypes
import functools
import hashlib
import subprocess
import tempfile
from pathlib import Path
from typing import TYPE_CHECKING

if TYPE_CHECKING:
    import torch

PACKAGE = Path(__file__).resolve().parent
KERNELS = PACKAGE / "csrc"
INCLUDE = PACKAGE.parent / "include"
NATIVE = PACKAGE / "_native"
HEAD_DIM = 128
LIBRARIES = ("kv_append", "decode_attn", "decode_step", "stream_gemm", "tile_gemm")

c_ptr, c_int, c_ll, c_float = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
SIGNATURES = {
    "kv_append": {
        "ncb_status_string": ([c_int], ctypes.c_char_p),
        "kv_cache_bytes": ([c_int, c_int, c_int], c_ll),
        "kv_cache_pages": ([c_int], c_int),
        "kv_append_fp8": ([c_ptr] * 9 + [c_ll, c_int, c_int, c_ll, c_int, c_int, c_int, c_ptr, c_ptr], c_int),
        "kv_append_fp8_ve": ([c_ptr] * 9 + [c_ll, c_int, c_int, c_ll, c_int, c_int, c_int] + [c_ptr] * 4
                             + [c_int, c_int, c_ptr, c_ptr], c_int),
    },
    "decode_attn": {
        "decode_attn_chunk_pages": ([c_int, c_int, c_int], c_int),
        "decode_attn_plan_chunk_pages": ([c_ptr, c_int, c_int, c_int, c_int], c_int),
        "decode_attn_workspace_bytes": ([c_int, c_int, c_int, c_int, c_int], c_ll),
        "decode_attn_fp8": ([c_ptr] * 5 + [c_ll, c_ptr] + [c_int] * 8 + [c_float, c_ptr, c_ptr], c_int),
        "decode_attn_fp8_partial": ([c_ptr] * 5 + [c_ll, c_ptr] + [c_int] * 8 + [c_float, c_ptr, c_ptr], c_int),
        "decode_attn_fp8_static": ([c_ptr] * 5 + [c_int] * 8 + [c_float, c_ptr, c_ptr], c_int),
        "decode_step_attn_fp8": ([c_ptr] * 9 + [c_ll, c_ptr, c_int, c_int, c_int, c_ll] + [c_int] * 6
                                 + [c_float, c_ptr, c_ptr], c_int),
        "decode_step_attn_fp8_ve": ([c_ptr] * 9 + [c_ll, c_ptr, c_int, c_int, c_int, c_ll] + [c_int] * 6
                                    + [c_float] + [c_ptr] * 4 + [c_int, c_int, c_ptr, c_ptr], c_int),
        "prefill_attn_rows_per_block": ([c_int, c_int], c_int),
        "prefill_attn_fp8": ([c_ptr] * 6 + [c_int, c_ptr, c_ll] + [c_int] * 4 + [c_float, c_ptr, c_ptr], c_int),
        "decode_attn_fp8_split": ([c_ptr] * 5 + [c_ll] + [c_int] * 8 + [c_float, c_ptr, c_ptr], c_int),
        "decode_attn_merge": ([c_ptr, c_int, c_ll, c_ptr, c_ptr], c_int),
        "decode_attn_fp8_sharded": ([c_ptr] * 5 + [c_ll, c_ptr] + [c_int] * 8 + [c_float, c_ptr, c_int, c_int, c_ptr,
                                                                               c_ptr, c_ptr], c_int),
    },
    "decode_step": {
        "skinny_gemm": ([c_ptr] * 4 + [c_int] * 5 + [c_ptr], c_int),
        "skinny_gemm_supported": ([c_int] * 4, c_int),
        "skinny_gemm_mix": ([c_ptr] * 4 + [c_float, c_float, c_ptr] + [c_int] * 4 + [c_ptr], c_int),
        "embed_norm": ([c_ptr] * 3 + [c_int] * 3 + [c_ptr], c_int),
        "embed_norm_mix": ([c_ptr] * 4 + [c_float, c_float] + [c_int] * 3 + [c_ptr], c_int),
        "add_rms_norm": ([c_ptr] * 3 + [c_ll, c_int, c_ptr], c_int),
        "add_rms_norm_mix": ([c_ptr] * 3 + [c_float, c_float, c_ptr, c_ll, c_int, c_ptr], c_int),
        "relu2_inplace": ([c_ptr, c_ll, c_ptr], c_int),
        "sample_choice": ([c_ptr] * 7 + [c_float, c_ptr, c_ptr, c_int, c_int, c_ptr, c_int, c_ptr], c_int),
        "greedy_choice": ([c_ptr] * 3 + [c_int] * 2 + [c_ptr, c_int, c_ptr], c_int),
    },
    "tile_gemm": {
        "tile_gemm": ([c_ptr] * 4 + [c_ll, c_int, c_int, c_int, c_ptr, c_ptr], c_int),
        "tile_gemm_form": ([c_ptr] * 4 + [c_ll, c_int, c_int, c_int, c_int, c_ptr, c_ptr], c_int),
    },
    "stream_gemm": {
        "stream_gemm_split": ([c_int, c_int, c_int], c_int),
        "stream_gemm": ([c_ptr] * 4 + [c_int] * 6 + [c_ptr, c_ll, c_ptr, c_ptr], c_int),
        "stream_gemm_mix": ([c_ptr] * 4 + [c_float, c_float, c_ptr] + [c_int] * 5 + [c_ptr, c_ll, c_ptr, c_ptr], c_int),
    },
}
STATUS = {0: "ok", 1: "invalid argument", 2: "misaligned pointer or stride", 3: "workspace too small",
          4: "kernel launch failed", 5: "unsupported shape (head ratio, tile width)", 6: "needs more than the built-in scratch"}


class NativeError(RuntimeError):
    """A native entry point returned a non-zero status."""


def command() -> list[str]:
    """The nvcc command, up to the output path."""
    return ["nvcc", "-gencode=arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-Xcompiler", "-fPIC", "-shared",
            "-o"]


def library_path(name: str) -> Path:
    """_native/<name>-<sha256(command, source, headers)>.so; the file may not exist yet."""
    digest = hashlib.sha256(" ".join(command()).encode())
    for source in [KERNELS / f"{name}.cu", *sorted(KERNELS.glob("*.cuh")), *sorted(INCLUDE.glob("*.h"))]:
        digest.update(source.read_bytes())
    return NATIVE / f"{name}-{digest.hexdigest()[:32]}.so"


def build_library(name: str) -> Path:
    """Build csrc/<name>.cu unless its cached library exists; built in a temporary directory and renamed
    atomically so concurrent first builds never share a file (reference native.py:27-40)."""
    path = library_path(name)
    if not path.exists():
        NATIVE.mkdir(exist_ok=True)
        for stale in NATIVE.glob(f"{name}-*.so"):
            stale.unlink(missing_ok=True)
        with tempfile.TemporaryDirectory(dir=NATIVE) as tmp:
            built = Path(tmp) / path.name
            subprocess.run([*command(), str(built), str(KERNELS / f"{name}.cu")], check=True)
            built.replace(path)
    return path


@functools.cache
def cuda_library(name: str) -> ctypes.CDLL:
    """csrc/<name>.cu as a loaded library with argtypes set; built first if needed, loaded once per process."""
    lib = ctypes.CDLL(str(build_library(name)))
    for symbol, (argtypes, restype) in SIGNATURES[name].items():
        fn = getattr(lib, symbol)  # AttributeError if the library does not export what the header declares
        fn.argtypes, fn.restype = argtypes, restype
    return lib


def pointer(t: "torch.Tensor | None") -> ctypes.c_void_p:
    return ctypes.c_void_p(None if t is None else t.data_ptr())


def stream() -> ctypes.c_void_p:
    """The current CUDA stream of the current device, which the kernels launch on. (The raw handle straight from
    torch's C layer: a row pass makes a hundred launches, and building a torch.cuda.Stream object for each cost
    more host time than small passes spend on the device.)"""
    import torch

    return ctypes.c_void_p(torch._C._cuda_getCurrentRawStream(torch.cuda.current_device()))


def check(status: int, what: str) -> None:
    if status != 0:
        raise NativeError(f"{what}: status {status} ({STATUS.get(status, 'unknown')})")
