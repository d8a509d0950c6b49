"""Small data utilities, one sub-command each (the reference's tools/calculate-cifar10-mean.rs,
dump-array3d-header.rs, load-array3d.rs, test-lmdb.rs, test-varraydb.rs):

    python -m rembrandt_b200.cli.data_tools cifar10-mean  <data_batch.bin> <out.ndarray>
    python -m rembrandt_b200.cli.data_tools dump-header   <file.ndarray> [--dtype f32|u8]
    python -m rembrandt_b200.cli.data_tools load-array    <file.ndarray> [--dtype f32|u8]
    python -m rembrandt_b200.cli.data_tools test-lmdb     <env dir or data.mdb> [--limit N]
    python -m rembrandt_b200.cli.data_tools test-recorddb <prefix> [--limit N]
    python -m rembrandt_b200.cli.data_tools make-lmdb     <data_batch.bin> <out dir> [--limit N]

`make-lmdb` writes the images of a CIFAR-10 binary file as a Caffe image database (keys "%08d", values raw `Datum`
messages), which is what the `lmdb_caffe` source and the native database loader read.
"""
import argparse
import json
import sys

import numpy as np

from ..utils import blob


def cifar10_mean(args):
    from ..data.datasets import Cifar10DataSource, compute_mean
    src = Cifar10DataSource(args.data)
    mean = compute_mean(src)                       # [C, H, W] float32
    blob.write_array_file(args.out, mean, "f32")   # dims (W, H, C), as cifar10_mean_32x32x3.ndarray
    print(json.dumps({"samples": len(src), "dims": [mean.shape[2], mean.shape[1], mean.shape[0]],
                      "mean_of_mean": float(mean.mean()), "out": args.out}))


def dump_header(args):
    with open(args.file, "rb") as f:
        buf = f.read()
    off, n = 0, 0
    while off < len(buf):
        recs, off2 = blob.decode_records(buf, args.dtype, off, count=1)
        if not recs:
            break
        data, dims, tag = recs[0]
        print(json.dumps({"record": n, "offset": off, "dims": list(dims), "elements": int(data.size),
                          "tag": tag.hex() if isinstance(tag, (bytes, bytearray)) else str(tag)}))
        off, n = off2, n + 1


def load_array(args):
    arr = blob.read_array_file(args.file, args.dtype)
    print(json.dumps({"shape": list(arr.shape), "dtype": str(arr.dtype), "min": float(arr.min()), "max": float(arr.max()),
                      "mean": float(arr.mean())}))


def test_lmdb(args):
    from ..data.codecs import decode_caffe_datum
    from ..data.lmdb_reader import open_env
    with open_env(args.path) as env:
        print(json.dumps({"entries": len(env), "depth": env.depth, "page_size": env.psize}))
        for i, (k, v) in enumerate(env.items()):
            if i >= args.limit:
                break
            row = {"key": k.decode("latin1"), "value_bytes": len(v)}
            try:
                d = decode_caffe_datum(v)
                row.update({"channels": d["channels"], "height": d["height"], "width": d["width"], "label": d["label"],
                            "encoded": d["encoded"]})
            except ValueError:
                pass      # not a Datum message: report the key and size only
            print(json.dumps(row))


def test_recorddb(args):
    from ..data.recorddb import RecordDb
    db = RecordDb(args.prefix)
    print(json.dumps({"records": len(db), "episodes": None if db.episodes is None else int(len(db.episodes))}))
    for i in range(min(args.limit, len(db))):
        print(json.dumps({"record": i, "bytes": len(db[i])}))


def make_lmdb(args):
    import os
    from ..data.codecs import encode_caffe_datum
    from ..data.datasets import Cifar10DataSource
    from ..data.lmdb_reader import write_env
    src = Cifar10DataSource(args.data)
    n = len(src) if not args.limit else min(args.limit, len(src))
    items = []
    for i in range(n):
        img, label = src[i]
        c, h, w = img.shape
        items.append((b"%08d" % i, encode_caffe_datum(np.ascontiguousarray(img).tobytes(), c, h, w, int(label))))
    os.makedirs(args.out, exist_ok=True)
    write_env(args.out, items)
    print(json.dumps({"records": n, "out": args.out}))


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("cifar10-mean"); p.add_argument("data"); p.add_argument("out"); p.set_defaults(fn=cifar10_mean)
    for name, fn in (("dump-header", dump_header), ("load-array", load_array)):
        p = sub.add_parser(name); p.add_argument("file"); p.add_argument("--dtype", default="f32"); p.set_defaults(fn=fn)
    p = sub.add_parser("test-lmdb"); p.add_argument("path"); p.add_argument("--limit", type=int, default=5)
    p.set_defaults(fn=test_lmdb)
    p = sub.add_parser("test-recorddb"); p.add_argument("prefix"); p.add_argument("--limit", type=int, default=5)
    p.set_defaults(fn=test_recorddb)
    p = sub.add_parser("make-lmdb"); p.add_argument("data"); p.add_argument("out")
    p.add_argument("--limit", type=int, default=0); p.set_defaults(fn=make_lmdb)
    args = ap.parse_args(argv)
    args.fn(args)
    return 0


if __name__ == "__main__":
    sys.exit(main())
