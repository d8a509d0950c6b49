"""Dataset readers, shards, iterators and codecs (CPU)."""
import struct

import numpy as np
import pytest
import torch

from rembrandt_b200.data import (AsyncPoolDataIter, AsyncQueueDataIter, BatchIter, Cifar10DataSource,
                                 CyclicSampleDataIter, MnistDataSource, ParallelJoinDataIter, RandomSampleDataIter,
                                 RangeDataShard, SequentialSampleIter, SyntheticDataSource, TransformDataIter,
                                 compute_mean, cyclic_partition_shard, partition_shard)
from rembrandt_b200.data import codecs
from rembrandt_b200.utils import blob


def write_idx(path, arr):
    with open(path, "wb") as f:
        f.write(bytes([0, 0, 0x08, arr.ndim]))
        for d in arr.shape:
            f.write(struct.pack(">I", d))
        f.write(arr.tobytes())


def test_mnist_idx_reader(tmp_path):
    rng = np.random.default_rng(0)
    imgs = rng.integers(0, 256, (7, 5, 6), dtype=np.uint8)          # 7 images of height 5, width 6
    lbls = rng.integers(0, 10, (7,), dtype=np.uint8)
    write_idx(tmp_path / "img", imgs)
    write_idx(tmp_path / "lbl", lbls)
    src = MnistDataSource(str(tmp_path / "img"), str(tmp_path / "lbl"))
    assert len(src) == 7 and src.dims == (6, 5, 1)
    x, y = src[3]
    assert x.shape == (1, 5, 6) and np.array_equal(x[0], imgs[3]) and y == lbls[3]
    (tmp_path / "bad").write_bytes(b"\x01\x02\x03")
    with pytest.raises(ValueError):
        MnistDataSource(str(tmp_path / "bad"), str(tmp_path / "lbl"))


def test_cifar_reader_and_mean(tmp_path):
    rng = np.random.default_rng(1)
    recs = rng.integers(0, 256, (5, 3073), dtype=np.uint8)
    recs[:, 0] %= 10
    (tmp_path / "c.bin").write_bytes(recs.tobytes())
    src = Cifar10DataSource(str(tmp_path / "c.bin"))
    assert len(src) == 5 and src.dims == (32, 32, 3)
    x, y = src[2]
    assert y == recs[2, 0] and np.array_equal(x.reshape(-1), recs[2, 1:])
    imgs, lbls = src.batch(1, 3)
    assert np.array_equal(lbls, recs[1:4, 0]) and np.array_equal(imgs[0].reshape(-1), recs[1, 1:])
    mean = compute_mean(src)
    assert np.allclose(mean.reshape(-1), recs[:, 1:].astype(np.float64).mean(0), atol=1e-4)
    (tmp_path / "short.bin").write_bytes(b"\x00" * 100)
    with pytest.raises(ValueError):
        Cifar10DataSource(str(tmp_path / "short.bin"))


def test_synthetic_source_is_a_pure_function_of_seed_and_index():
    a, b = SyntheticDataSource(10, (8, 8, 3), 5, seed=3), SyntheticDataSource(10, (8, 8, 3), 5, seed=3)
    c = SyntheticDataSource(10, (8, 8, 3), 5, seed=4)
    assert np.array_equal(a[7][0], b[7][0]) and a[7][1] == b[7][1]
    assert not np.array_equal(a[7][0], c[7][0])
    assert a[0][0].shape == (3, 8, 8) and a[0][0].dtype == np.uint8


def test_shards_partition_the_source():
    src = list(range(10))
    shards = [partition_shard(src, r, 3) for r in range(3)]
    assert [list(SequentialSampleIter(s)) for s in shards] == [[0, 1, 2, 3], [4, 5, 6], [7, 8, 9]]
    wrap = cyclic_partition_shard(src, 0, 2, 7)
    assert list(SequentialSampleIter(wrap)) == [7, 8, 9, 0, 1]
    with pytest.raises(IndexError):
        RangeDataShard(src, 2, 4)[5]


def test_iterators():
    shard = RangeDataShard(list(range(20)))
    r1 = list(RandomSampleDataIter(shard, seed=(1, 2)))
    assert len(r1) == 20 and r1 == list(RandomSampleDataIter(shard, seed=(1, 2))) and set(r1) <= set(range(20))
    cyc = iter(CyclicSampleDataIter(RangeDataShard([1, 2, 3])))
    assert [next(cyc) for _ in range(7)] == [1, 2, 3, 1, 2, 3, 1]
    assert list(TransformDataIter(SequentialSampleIter(shard), lambda v: v + 1))[:3] == [1, 2, 3]
    aq = AsyncQueueDataIter(SequentialSampleIter(shard), capacity=4)
    assert list(aq) == list(range(20))
    assert list(aq) == list(range(20))                               # restartable
    assert list(AsyncPoolDataIter(range(50), lambda v: v * 2, num_workers=4, window=8)) == [2 * v for v in range(50)]
    assert sorted(ParallelJoinDataIter([range(0, 5), range(5, 9)])) == list(range(9))


def test_async_iterators_surface_producer_errors():
    def bad():
        yield 1
        raise RuntimeError("decode failed")
    with pytest.raises(RuntimeError, match="decode failed"):
        list(AsyncQueueDataIter(bad()))

    def boom(v):
        if v == 3:
            raise ValueError("bad sample")
        return v
    with pytest.raises(ValueError, match="bad sample"):
        list(AsyncPoolDataIter(range(6), boom, 2))


def test_batch_iter_packs_samples():
    src = SyntheticDataSource(10, (4, 4, 1), 3, seed=0)
    batches = list(BatchIter(SequentialSampleIter(RangeDataShard(src)), 4, src.dims, depth=2))
    assert len(batches) == 2
    x, y = batches[1]
    assert x.shape == (4, 1, 4, 4) and x.dtype == torch.uint8 and y.dtype == torch.int32
    assert np.array_equal(x[1].numpy(), src[5][0]) and int(y[1]) == src[5][1]


def test_codecs_and_caffe_datum():
    img = np.arange(24, dtype=np.uint8).reshape(2, 3, 4)             # [c][h][w]
    rec = blob.encode_record(img.reshape(-1), (4, 3, 2), dtype="u8")
    assert np.array_equal(codecs.Array3dDataCodec().decode(rec), img)
    assert codecs.FakeJpegDataCodec().decode(b"whatever").shape == (3, 256, 256)
    # hand-assembled Datum: channels=2, height=3, width=4, data, label=7
    msg = b"\x08\x02\x10\x03\x18\x04" + b"\x22" + bytes([24]) + img.tobytes() + b"\x28\x07"
    d = codecs.decode_caffe_datum(msg)
    assert (d["channels"], d["height"], d["width"], d["label"], d["encoded"]) == (2, 3, 4, 7, False)
    x, y = codecs.datum_to_sample(d)
    assert np.array_equal(x, img) and y == 7
    assert np.array_equal(codecs.transpose_whc_to_cwh(codecs.transpose_cwh_to_whc(img)), img)
    crop, _ = codecs.CenterCropPreproc(2, 1)((img, 0))
    assert np.array_equal(crop, img[:, 1:2, 1:3])
    rc, _ = codecs.RandomCropPreproc(2, 2, seed=1)((img, 0))
    assert rc.shape == (2, 2, 2)


def test_lmdb_reader_round_trip_with_depth_and_overflow(tmp_path):
    """The dependency-free LMDB reader: ordered iteration, get, cursor seek, overflow values, multi-level tree."""
    import random
    from rembrandt_b200.data.lmdb_reader import LmdbEnv, NativeLmdbEnv, write_env
    rnd = random.Random(5)
    items = []
    for i in range(700):
        key = b"%08d" % i
        size = rnd.choice([0, 1, 17, 300, 900, 5000, 20000]) if i % 7 == 0 else rnd.randint(1, 200)
        items.append((key, bytes(rnd.getrandbits(8) for _ in range(size))))
    for cap in (0, 5):           # natural fan-out, and 5 nodes per page (a tree of depth >= 4)
        d = tmp_path / f"db{cap}"
        write_env(str(d), items, max_leaf_nodes=cap)
        for cls in (LmdbEnv, NativeLmdbEnv):     # the Python reader and the C++ cursor must agree
            with cls(str(d)) as env:
                assert len(env) == 700
                if cap:
                    assert env.depth >= 4
                got = list(env.items())
                assert got == sorted(items)
                assert env.get(b"00000123") == dict(items)[b"00000123"]
                assert env.get(b"00000699") == dict(items)[b"00000699"]
                assert env.get(b"nope") is None
                tail = list(env.items(b"00000650"))
                assert [k for k, _ in tail] == [b"%08d" % i for i in range(650, 700)]
                assert next(iter(env.items(b"000001235")))[0] == b"00000124"   # seek lands on the next larger key


def test_lmdb_caffe_shard_partitions_and_decodes(tmp_path):
    from rembrandt_b200.data.codecs import encode_caffe_datum
    from rembrandt_b200.data.lmdb_reader import LmdbCaffeShard, write_env
    rng = np.random.default_rng(0)
    imgs = [rng.integers(0, 256, (3, 8, 6), dtype=np.uint8) for _ in range(10)]
    items = [(b"%08d_img" % i, encode_caffe_datum(imgs[i].tobytes(), 3, 8, 6, label=i * 3)) for i in range(10)]
    write_env(str(tmp_path / "db"), items)
    seen = []
    for rank in range(3):
        shard = LmdbCaffeShard(str(tmp_path / "db"), rank, 3)
        for img, label in shard:
            seen.append(label // 3)
            assert np.array_equal(img, imgs[label // 3])
    assert seen == list(range(10))


def test_record_stores_shards_and_episode_lookahead(tmp_path):
    import struct
    from rembrandt_b200.data.codecs import Array3dDataCodec
    from rembrandt_b200.data.recorddb import EpisodeDataSource, RecordDb, RecordDbWriter, VarrayDbShard
    from rembrandt_b200.utils import blob
    rng = np.random.default_rng(1)
    imgs = [rng.integers(0, 256, (2, 3 + i % 3, 4), dtype=np.uint8) for i in range(9)]
    with RecordDbWriter(str(tmp_path / "d")) as wd, RecordDbWriter(str(tmp_path / "l")) as wl:
        for i, im in enumerate(imgs):
            wd.append(blob.encode_record(im.reshape(-1), tuple(reversed(im.shape)), dtype="u8"))
            wl.append(struct.pack("<i", 100 + i))
    db = RecordDb(str(tmp_path / "d"))
    assert len(db) == 9
    got = []
    for rank in range(2):
        shard = VarrayDbShard(str(tmp_path / "d"), str(tmp_path / "l"), Array3dDataCodec(), rank, 2)
        for im, label in shard:
            assert np.array_equal(im, imgs[label - 100])
            got.append(label - 100)
    assert got == list(range(9))
    # episodes of Go-like frames: label -1 marks a frame without a target
    labels = [[3, 5, -1, 7], [2, 9]]
    with RecordDbWriter(str(tmp_path / "e")) as we:
        for ep in labels:
            we.append_episode([struct.pack("<i", l) + bytes([l & 0xFF if l >= 0 else 0] * 9) for l in ep])
    src = EpisodeDataSource(str(tmp_path / "e"), (3, 3, 1), lookahead=3)
    assert len(src) == 5
    frame, la = src[0]
    assert frame.shape == (1, 3, 3) and la == [3, 5, -1]
    assert src[2][1] == [7, -1, -1]          # the frame after the unlabeled one; its episode ends
    assert src[3][1] == [2, 9, -1]


def test_data_tools_cli(tmp_path, capsys):
    import json
    from rembrandt_b200.cli import data_tools
    from rembrandt_b200.data.lmdb_reader import write_env
    from rembrandt_b200.data.codecs import encode_caffe_datum
    from rembrandt_b200.utils import blob
    # a CIFAR-10 style file of 7 records (1 label byte + 3072 pixel bytes)
    rng = np.random.default_rng(2)
    recs = rng.integers(0, 256, (7, 3073), dtype=np.uint8)
    (tmp_path / "batch.bin").write_bytes(recs.tobytes())
    data_tools.main(["cifar10-mean", str(tmp_path / "batch.bin"), str(tmp_path / "mean.ndarray")])
    out = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert out["samples"] == 7 and out["dims"] == [32, 32, 3]
    mean = blob.read_array_file(str(tmp_path / "mean.ndarray"), "f32")
    want = recs[:, 1:].astype(np.float64).mean(0).reshape(3, 32, 32)
    assert np.allclose(mean, want, atol=1e-3)
    data_tools.main(["dump-header", str(tmp_path / "mean.ndarray")])
    hdr = json.loads(capsys.readouterr().out.strip().splitlines()[0])
    assert hdr["dims"] == [32, 32, 3] and hdr["elements"] == 3072
    data_tools.main(["load-array", str(tmp_path / "mean.ndarray")])
    assert json.loads(capsys.readouterr().out.strip())["shape"] == [3, 32, 32]
    write_env(str(tmp_path / "db"), [(b"%08d" % i, encode_caffe_datum(bytes(12), 3, 2, 2, label=i)) for i in range(4)])
    data_tools.main(["test-lmdb", str(tmp_path / "db"), "--limit", "2"])
    lines = capsys.readouterr().out.strip().splitlines()
    assert json.loads(lines[0])["entries"] == 4 and json.loads(lines[2])["label"] == 1


@pytest.mark.parametrize("mode,threads", [("cyclic", 1), ("cyclic", 4), ("random", 3), ("shuffled", 4)])
def test_native_batch_loader_order_is_deterministic_and_sharded(mode, threads):
    from rembrandt_b200.data.native_loader import NativeBatchLoader
    n, batch = 103, 8
    images = (np.arange(n, dtype=np.uint32)[:, None, None, None] * np.ones((1, 2, 3, 3), dtype=np.uint32) % 251).astype(np.uint8)
    labels = np.arange(n, dtype=np.int32) + 1000
    lo, hi = 10, 93
    runs = []
    for _ in range(2):
        ld = NativeBatchLoader(images, labels, batch, mode=mode, seed=7, threads=threads, slots=5, shard=(lo, hi),
                               pin=False, max_batches=40)
        seen = []
        for k, (im, lb) in enumerate(ld):
            idx = lb.numpy() - 1000
            assert ((idx >= lo) & (idx < hi)).all()
            assert np.array_equal(im.numpy().reshape(batch, -1)[:, 0], images[idx].reshape(batch, -1)[:, 0])
            assert [ld.sample_index(k * batch + i) for i in range(batch)] == idx.tolist()
            seen.append(idx.copy())
        ld.close()
        assert len(seen) == 40
        runs.append(np.concatenate(seen))
    assert np.array_equal(runs[0], runs[1]), "order must not depend on thread timing"
    flat = runs[0]
    if mode == "cyclic":
        assert np.array_equal(flat, lo + np.arange(flat.size) % (hi - lo))
    if mode == "shuffled":
        ep = hi - lo
        for e in range(flat.size // ep):
            assert sorted(flat[e * ep:(e + 1) * ep].tolist()) == list(range(lo, hi)), "every epoch is a permutation"
        assert not np.array_equal(flat[:ep], flat[ep:2 * ep])
    if mode == "random":
        assert len(set(flat.tolist())) > (hi - lo) // 2


def test_bit_plane_codecs_round_trip():
    from rembrandt_b200.data import codecs
    from rembrandt_b200.utils import blob
    rng = np.random.default_rng(0)
    bits = rng.integers(0, 2, (5, 19, 19))
    planes = rng.integers(0, 256, (3, 19, 19)).astype(np.uint8)
    rec = codecs.BitsThenBytes3dCodec.encode(bits, planes)
    assert len(rec) == 32 + (5 * 361 + 7) // 8 + 32 + 3 * 361        # two headers, packed bits, bytes
    out = codecs.BitsThenBytes3dCodec(255).decode(rec)
    assert out.shape == (8, 19, 19) and (out[:5] == bits * 255).all() and (out[5:] == planes).all()
    assert (codecs.Bits3dCodec(7).decode(codecs.encode_bits3d(bits)) == bits * 7).all()
    with pytest.raises(blob.BlobError):
        codecs.Bits3dCodec().decode(rec[:40])
    with pytest.raises(blob.BlobError):
        codecs.Bits3dCodec().decode(blob.encode_record(planes.reshape(-1), (19, 19, 3), "u8"))   # not a bit record


def test_episode_iterators_partition_and_augment(tmp_path):
    import struct
    from collections import Counter
    from rembrandt_b200.data import (AugmentDataSource, CyclicEpisodeIterator, PartitionDataSource,
                                     RandomEpisodeIterator, SampleIterator, episode_ranges)
    from rembrandt_b200.data.recorddb import EpisodeDataSource, RecordDbWriter
    # three games of 6, 2 and 4 labelled positions (labels double as position ids); one unlabelled frame in game 0
    games = [[0, 1, 2, -1, 3, 4, 5], [10, 11], [20, 21, 22, 23]]
    with RecordDbWriter(str(tmp_path / "e")) as we:
        for ep in games:
            we.append_episode([struct.pack("<i", l) + bytes(9) for l in ep])
    src = EpisodeDataSource(str(tmp_path / "e"), (3, 3, 1))
    assert len(src) == 12 and src.episode_ranges() == [(0, 6), (6, 8), (8, 12)]
    assert [lab for _, lab in SampleIterator(src)] == [0, 1, 2, 3, 4, 5, 10, 11, 20, 21, 22, 23]
    # random episodes: each game is drawn about equally often although their lengths differ 3 : 1 : 2
    it = RandomEpisodeIterator(src, seed=(5, 6))
    draws = [lab // 10 for _ in range(100) for _, lab in it]
    c = Counter(draws)
    assert len(draws) == 1200 and all(330 < c[g] < 470 for g in range(3)), c
    # cyclic: games in order, one position of each, until len(source) positions
    cyc = [lab // 10 for _, lab in CyclicEpisodeIterator(src, seed=(7, 8))]
    assert cyc == [0, 1, 2] * 4
    # a source without episodes: one episode per sample
    plain = SyntheticDataSource(5, (4, 4, 1), 3, seed=0)
    assert episode_ranges(plain) == [(i, i + 1) for i in range(5)]
    assert len(list(RandomEpisodeIterator(plain))) == 5
    # partitions cut at game boundaries
    parts = [PartitionDataSource(r, 2, src) for r in range(2)]
    assert [len(p) for p in parts] == [8, 4] or [len(p) for p in parts] == [6, 6]
    assert sorted(lab for p in parts for _, lab in SampleIterator(p)) == sorted(l for g in games for l in g if l >= 0)
    for p in parts:
        for lo, hi in p.episode_ranges():
            assert len({p[i][1] // 10 for i in range(lo, hi)}) == 1     # an episode holds one game
    assert [len(PartitionDataSource(r, 2, plain)) for r in range(2)] == [3, 2]
    # host-side augmentation keeps the episode structure
    aug = AugmentDataSource(lambda im, lab: (im + 1, lab), src)
    assert len(aug) == 12 and aug.episode_ranges() == src.episode_ranges()
    assert int(aug[0][0].max()) == 1 and aug[3][1] == 3


def test_native_loader_over_a_caffe_database(tmp_path):
    from rembrandt_b200.data.codecs import encode_caffe_datum
    from rembrandt_b200.data.lmdb_reader import write_env
    from rembrandt_b200.data.native_loader import NativeBatchLoader
    rng = np.random.default_rng(4)
    imgs = rng.integers(0, 256, (37, 3, 5, 4), dtype=np.uint8)
    items = [(b"%08d" % i, encode_caffe_datum(imgs[i].tobytes(), 3, 5, 4, label=100 + i)) for i in range(37)]
    write_env(str(tmp_path), items, max_leaf_nodes=5)
    ld = NativeBatchLoader.from_caffe_lmdb(str(tmp_path), (3, 5, 4), batch=6, mode="cyclic", threads=3, pin=False,
                                           max_batches=13)
    seen = []
    for x, y in ld:
        assert x.shape == (6, 3, 5, 4)
        for j in range(6):
            i = int(y[j]) - 100
            assert np.array_equal(x[j].numpy(), imgs[i])
            seen.append(i)
    ld.close()
    assert seen == [k % 37 for k in range(78)]
    # a shard of records 10 .. 19, shuffled epochs: every record of the shard once per epoch
    ld = NativeBatchLoader.from_caffe_lmdb(str(tmp_path), (3, 5, 4), batch=5, mode="shuffled", seed=3, threads=2,
                                           shard=(10, 20), pin=False, max_batches=4)
    got = [int(v) - 100 for _, y in ld for v in y]
    ld.close()
    assert sorted(got[:10]) == list(range(10, 20)) and sorted(got[10:]) == list(range(10, 20))
    with pytest.raises(RuntimeError, match="not of the given shape"):
        NativeBatchLoader.from_caffe_lmdb(str(tmp_path), (3, 5, 5), batch=2, pin=False)
    with pytest.raises(RuntimeError, match="cannot open"):
        NativeBatchLoader.from_caffe_lmdb(str(tmp_path / "missing"), (3, 5, 4), batch=2, pin=False)


def test_make_lmdb_tool_round_trips_a_cifar_file(tmp_path, capsys):
    import json
    from rembrandt_b200.cli import data_tools
    from rembrandt_b200.data.lmdb_reader import LmdbCaffeShard
    from rembrandt_b200.data.native_loader import NativeBatchLoader
    rng = np.random.default_rng(6)
    recs = rng.integers(0, 256, (9, 3073), dtype=np.uint8)
    recs[:, 0] %= 10
    (tmp_path / "batch.bin").write_bytes(recs.tobytes())
    data_tools.main(["make-lmdb", str(tmp_path / "batch.bin"), str(tmp_path / "db")])
    assert json.loads(capsys.readouterr().out.strip().splitlines()[-1])["records"] == 9
    got = list(LmdbCaffeShard(str(tmp_path / "db")))
    assert len(got) == 9
    for i, (img, label) in enumerate(got):
        assert label == int(recs[i, 0]) and np.array_equal(img.reshape(-1), recs[i, 1:])
    ld = NativeBatchLoader.from_caffe_lmdb(str(tmp_path / "db"), (3, 32, 32), batch=3, mode="cyclic", pin=False,
                                           max_batches=3)
    labels = [int(v) for _, y in ld for v in y]
    ld.close()
    assert labels == [int(v) for v in recs[:, 0]]


def test_jpeg_records_decode_through_the_database_shards(tmp_path):
    """Encoded (JPEG) image records of a Caffe database and of a record store, decoded through Pillow: planar RGB out,
    grey images replicated to three channels."""
    PIL = pytest.importorskip("PIL.Image")
    import io
    import struct
    from rembrandt_b200.data.codecs import JpegDataCodec, encode_caffe_datum
    from rembrandt_b200.data.lmdb_reader import LmdbCaffeShard, write_env
    from rembrandt_b200.data.recorddb import RecordDbWriter, VarrayDbShard
    rng = np.random.default_rng(8)

    def jpeg(arr, mode):
        buf = io.BytesIO()
        PIL.fromarray(arr, mode).save(buf, format="JPEG", quality=95)
        return buf.getvalue()
    # smooth images survive JPEG closely enough to be recognised
    ramp = np.linspace(0, 255, 24 * 20).reshape(24, 20)
    colour = np.stack([ramp, ramp[::-1], ramp * 0.5], axis=2).astype(np.uint8)
    grey = ramp.astype(np.uint8)
    blobs = [jpeg(colour, "RGB"), jpeg(grey, "L")]
    codec = JpegDataCodec()
    out = codec.decode(blobs[0])
    assert out.shape == (3, 24, 20) and np.abs(out.astype(int) - colour.transpose(2, 0, 1).astype(int)).mean() < 6
    g3 = codec.decode(blobs[1])
    assert g3.shape == (3, 24, 20) and np.array_equal(g3[0], g3[1]) and np.abs(g3[0].astype(int) - grey).mean() < 4
    # Caffe database with encoded records
    (tmp_path / "db").mkdir()
    write_env(str(tmp_path / "db"), [(b"%08d" % i, encode_caffe_datum(b, 3, 24, 20, label=5 + i, encoded=True))
                                     for i, b in enumerate(blobs)])
    got = list(LmdbCaffeShard(str(tmp_path / "db"), codec=codec))
    assert [lab for _, lab in got] == [5, 6] and got[0][0].shape == (3, 24, 20)
    # record store (value blobs + little-endian labels)
    with RecordDbWriter(str(tmp_path / "d")) as wd, RecordDbWriter(str(tmp_path / "l")) as wl:
        for i, b in enumerate(blobs):
            wd.append(b)
            wl.append(struct.pack("<i", 40 + i))
    rows = list(VarrayDbShard(str(tmp_path / "d"), str(tmp_path / "l"), codec))
    assert [lab for _, lab in rows] == [40, 41] and np.array_equal(rows[1][0], g3)


def test_numa_binding_reads_the_topology_from_sysfs(tmp_path):
    """The rank-to-NUMA-node binding parses a (fake) sysfs tree; nothing is changed when the topology is unreadable."""
    import os
    from rembrandt_b200.utils import numa
    d = str(tmp_path)
    os.makedirs(f"{d}/bus/pci/devices/0000:1b:00.0")
    open(f"{d}/bus/pci/devices/0000:1b:00.0/numa_node", "w").write("1\n")
    os.makedirs(f"{d}/devices/system/node/node1")
    open(f"{d}/devices/system/node/node1/cpulist", "w").write("0-1,3\n")
    assert numa.numa_node_of_bus("0000:1B:00.0", d) == 1
    assert numa.node_cpus(1, d) == [0, 1, 3]
    assert numa._parse_cpulist("0-3,8,10-11") == [0, 1, 2, 3, 8, 10, 11]
    assert numa.numa_node_of_bus("0000:ff:00.0", d) is None and numa.node_cpus(7, d) == []
    open(f"{d}/bus/pci/devices/0000:1b:00.0/numa_node", "w").write("-1\n")      # single-node machine
    assert numa.numa_node_of_bus("0000:1b:00.0", d) is None
    assert numa.bind_to_gpu_node(0, sysfs=str(tmp_path / "absent")) is None
