"""Packer throughput: documents of random length packed into fixed-length rows, every packer on the same corpus.

    python -m benchmarks.bench_packers [--docs 2000] [--seq-len 4096]

Mirrors the micro-benchmark of the reference's packing suite (``tests/dataloader_packing.py:160-185,251-279``):
warm-up runs, garbage collection off inside the timed repeats, median / minimum / spread per packer, rows produced
and padding fraction.  CPU only.
"""

from __future__ import annotations

import argparse
import gc
import json
import random
import time
from statistics import median, pstdev


def make_corpus(n_docs: int, seq_len: int, seed: int = 0) -> list[list[int]]:
    rng = random.Random(seed)
    docs = []
    for _ in range(n_docs):
        n = max(1, min(seq_len, int(rng.lognormvariate(6.0, 1.0))))
        docs.append([rng.randrange(1, 50000) for _ in range(n)])
    return docs


def bench(fn, warmup: int = 2, repeats: int = 7):
    out = None
    for _ in range(warmup):
        out = fn()
    samples = []
    was = gc.isenabled()
    gc.disable()
    try:
        for _ in range(repeats):
            t0 = time.perf_counter()
            out = fn()
            samples.append(time.perf_counter() - t0)
    finally:
        if was:
            gc.enable()
    return out, median(samples), min(samples), (pstdev(samples) if len(samples) > 1 else 0.0)


def main(argv=None) -> None:
    from torchure_b200.data import packers as P

    ap = argparse.ArgumentParser()
    ap.add_argument("--docs", type=int, default=2000)
    ap.add_argument("--seq-len", type=int, default=4096)
    args = ap.parse_args(argv)
    docs = make_corpus(args.docs, args.seq_len)
    n_tokens = sum(len(d) for d in docs)
    rows = []
    registry = {**P.PACKERS, **P.BESTFIT_PACKERS}
    for name in sorted(registry):
        packer = registry[name](None, seq_len=args.seq_len, eos_id=0, pad_id=0)
        out, med, best, spread = bench(lambda: packer.pack_to_tensor(docs))
        n_rows = int(out.shape[0])
        rows.append({"packer": name, "median_s": med, "min_s": best, "stdev_s": spread, "rows": n_rows,
                     "tokens_per_s": n_tokens / med,
                     "rows_fill": (n_tokens + len(docs)) / max(1, n_rows * args.seq_len)})
    print(json.dumps({"docs": args.docs, "tokens": n_tokens, "seq_len": args.seq_len, "results": rows}, indent=1))


if __name__ == "__main__":
    main()
