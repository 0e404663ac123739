"""Builds the C checker oracle/_build/libzck_oracle.so with gcc (test infrastructure; never part of the product)."""

import pathlib
import subprocess

HERE = pathlib.Path(__file__).resolve().parent
OUT = HERE / "_build" / "libzck_oracle.so"


def build():
    source = HERE / "quant_rules.c"
    if OUT.exists() and OUT.stat().st_mtime >= source.stat().st_mtime:
        return OUT
    OUT.parent.mkdir(exist_ok=True)
    # -ffp-contract=off and no fast-math: every operation rounds as written
    subprocess.run(["gcc", "-O2", "-std=c11", "-shared", "-fPIC", "-ffp-contract=off", "-fno-fast-math", "-o", str(OUT),
                    str(source), "-lm"], check=True)
    return OUT


if __name__ == "__main__":
    print(build())
