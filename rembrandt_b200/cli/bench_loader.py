"""bench-loader: how many images per second the host side can assemble into batches (no GPU involved).

Compares the C++ prefetching loader (worker threads filling a ring of slots, `--threads`) with the Python iterator
chain (`RandomSampleDataIter` -> `AsyncQueueDataIter` -> `BatchIter`) on an in-memory uint8 dataset of the given sample
shape. The training step consumes `images/s x bytes per image`; the loader has to stay above that.

    python -m rembrandt_b200.cli.bench_loader --shape 3 227 227 --batch 128 --threads 1 4 8
"""
import argparse
import json
import time

import numpy as np

from ..data import AsyncQueueDataIter, BatchIter, RandomSampleDataIter, RangeDataShard
from ..data.native_loader import NativeBatchLoader


class _Arrays:
    def __init__(self, images, labels):
        self.images, self.labels = images, labels
        c, h, w = images.shape[1:]
        self.dims = (w, h, c)

    def __len__(self):
        return len(self.images)

    def __getitem__(self, i):
        return self.images[i], int(self.labels[i])


def measure(shape, samples, batch, batches, threads_list):
    rng = np.random.default_rng(0)
    images = rng.integers(0, 256, (samples,) + tuple(shape), dtype=np.uint8)
    labels = rng.integers(0, 1000, samples).astype(np.int32)
    per_image = int(np.prod(shape))
    rows = []
    for threads in threads_list:
        ld = NativeBatchLoader(images, labels, batch, mode="shuffled", threads=threads, slots=6, pin=False)
        for _ in range(3):
            next(ld)
        t0 = time.perf_counter()
        for _ in range(batches):
            next(ld)
        dt = time.perf_counter() - t0
        ld.close()
        rows.append({"loader": f"native x{threads}", "images_per_s": batches * batch / dt,
                     "gb_per_s": batches * batch * per_image / dt / 1e9})
    src = _Arrays(images, labels)
    it = iter(BatchIter(AsyncQueueDataIter(_forever(RandomSampleDataIter(RangeDataShard(src)))), batch, src.dims))
    for _ in range(3):
        next(it)
    n = max(2, batches // 8)
    t0 = time.perf_counter()
    for _ in range(n):
        next(it)
    dt = time.perf_counter() - t0
    rows.append({"loader": "python iterators", "images_per_s": n * batch / dt, "gb_per_s": n * batch * per_image / dt / 1e9})
    return rows


def measure_lmdb(shape, samples, batch, batches, threads_list):
    """The same comparison over a Caffe image database written to a temporary directory: the C++ loader reading the
    memory-mapped environment against the Python cursor + `Datum` decode (`LmdbCaffeShard`)."""
    import tempfile
    from ..data.codecs import encode_caffe_datum
    from ..data.lmdb_reader import LmdbCaffeShard, write_env
    rng = np.random.default_rng(0)
    c, h, w = shape
    per_image = c * h * w
    rows = []
    with tempfile.TemporaryDirectory() as d:
        write_env(d, [(b"%08d" % i, encode_caffe_datum(rng.integers(0, 256, per_image, dtype=np.uint8).tobytes(), c, h, w,
                                                       label=i % 1000)) for i in range(samples)])
        for threads in threads_list:
            ld = NativeBatchLoader.from_caffe_lmdb(d, (c, h, w), batch, mode="shuffled", threads=threads, slots=6, pin=False)
            for _ in range(3):
                next(ld)
            t0 = time.perf_counter()
            for _ in range(batches):
                next(ld)
            dt = time.perf_counter() - t0
            ld.close()
            rows.append({"loader": f"native lmdb x{threads}", "images_per_s": batches * batch / dt,
                         "gb_per_s": batches * batch * per_image / dt / 1e9})
        t0 = time.perf_counter()
        n = sum(1 for _ in LmdbCaffeShard(d))
        dt = time.perf_counter() - t0
        rows.append({"loader": "python lmdb cursor", "images_per_s": n / dt, "gb_per_s": n * per_image / dt / 1e9})
    return rows


def _forever(it):
    while True:
        for x in it:
            yield x


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--shape", type=int, nargs=3, default=[3, 227, 227], metavar=("C", "H", "W"))
    ap.add_argument("--samples", type=int, default=2048)
    ap.add_argument("--batch", type=int, default=128)
    ap.add_argument("--batches", type=int, default=64)
    ap.add_argument("--threads", type=int, nargs="+", default=[1, 2, 4, 8])
    ap.add_argument("--lmdb", action="store_true", help="read the samples from a Caffe image database instead of arrays")
    args = ap.parse_args(argv)
    fn = measure_lmdb if args.lmdb else measure
    rows = fn(args.shape, args.samples, args.batch, args.batches, args.threads)
    for r in rows:
        print(f"{r['loader']:<18s} {r['images_per_s']:12.0f} images/s {r['gb_per_s']:8.2f} GB/s")
    print(json.dumps({"shape": args.shape, "batch": args.batch, "rows": rows}))
    return rows


if __name__ == "__main__":
    main()
