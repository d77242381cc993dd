"""Compile oracle/kv_append_oracle.c into oracle/_build/libkv_append_oracle.so (test infrastructure).

-ffp-contract=off keeps every fp32 operation individually rounded, which is what makes the CPU bits comparable
to the GPU kernel's __f*_rn arithmetic. Run as a script or call build()."""

import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
SOURCE = HERE / "kv_append_oracle.c"
OUTPUT = HERE / "_build" / "libkv_append_oracle.so"
COMMAND = ["gcc", "-O2", "-ffp-contract=off", "-fno-fast-math", "-fPIC", "-shared", "-o"]


def build(force: bool = False) -> Path:
    """The shared object, rebuilt when the source is newer."""
    if force or not OUTPUT.exists() or OUTPUT.stat().st_mtime < SOURCE.stat().st_mtime:
        OUTPUT.parent.mkdir(exist_ok=True)
        tmp = OUTPUT.with_suffix(".tmp.so")
        subprocess.run([*COMMAND, str(tmp), str(SOURCE), "-lm"], check=True)
        tmp.replace(OUTPUT)
    return OUTPUT


if __name__ == "__main__":
    print(build(force=True))
