#!/usr/bin/env python
"""Command line of the reference's Newton-Schulz benchmark (``--single --m M [--n N]``,
``--grid [--expansion E]``, ``--plot``, ``--batch_size B``), answered by
``bench_newton_schulz.py`` of this folder."""
import argparse
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def translate(argv):
    p = argparse.ArgumentParser(description=__doc__)
    mode = p.add_mutually_exclusive_group(required=True)
    mode.add_argument("--single", action="store_true")
    mode.add_argument("--grid", action="store_true")
    mode.add_argument("--plot", action="store_true")
    p.add_argument("--m", type=int)
    p.add_argument("--n", type=int)
    p.add_argument("--batch_size", type=int, default=1)
    p.add_argument("--expansion", type=int, default=1)
    p.add_argument("--dtype", default="bfloat16", choices=["bfloat16"])
    a = p.parse_args(argv)
    out = ["--batch", str(a.batch_size)]
    if a.single:
        if a.m is None:
            p.error("--single needs --m")
        return out + ["--single", str(a.m), str(a.n or a.m)]
    if a.grid:
        return out + ["--sweep", "--expansion", str(a.expansion)]
    return out + ["--curve"]


if __name__ == "__main__":
    sys.path.insert(0, HERE)
    import bench_newton_schulz

    sys.argv = [os.path.join(HERE, "bench_newton_schulz.py")] + translate(sys.argv[1:])
    bench_newton_schulz.main()
