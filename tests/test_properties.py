"""Property-based checks (hypothesis) of the host-side building blocks."""
import numpy as np
import pytest
from hypothesis import given, settings, strategies as st

from rembrandt_b200.utils import blob
from rembrandt_b200.utils.rng import cyclic_partition_range, partition_range


@settings(max_examples=60, deadline=None)
@given(st.lists(st.integers(1, 7), min_size=1, max_size=4), st.sampled_from(["f32", "u8"]), st.integers(0, 2**32 - 1))
def test_blob_records_round_trip(dims, dtype, seed):
    rng = np.random.default_rng(seed)
    n = int(np.prod(dims))
    data = rng.integers(0, 256, n).astype(np.uint8) if dtype == "u8" else rng.standard_normal(n).astype(np.float32)
    buf = blob.encode_record(data, tuple(dims), dtype=dtype) + blob.encode_record(data[::-1].copy(), (n,), dtype=dtype)
    recs, off = blob.decode_records(buf, dtype)
    assert off == len(buf) and len(recs) == 2
    assert tuple(recs[0][1]) == tuple(dims) and np.array_equal(recs[0][0], data)
    assert np.array_equal(recs[1][0], data[::-1])


@settings(max_examples=100, deadline=None)
@given(st.integers(0, 10_000), st.integers(1, 64))
def test_partition_range_is_a_balanced_contiguous_cover(n, parts):
    bounds = [partition_range(n, parts, i) for i in range(parts)]
    assert bounds[0][0] == 0 and bounds[-1][1] == n
    sizes = []
    for (lo, hi), (lo2, _hi2) in zip(bounds, bounds[1:] + [(n, n)]):
        assert lo <= hi and hi == lo2
        sizes.append(hi - lo)
    assert max(sizes) - min(sizes) <= 1


@settings(max_examples=60, deadline=None)
@given(st.integers(1, 500), st.integers(1, 8), st.integers(0, 1000))
def test_cyclic_partition_covers_every_element_once(n, parts, shift):
    seen = []
    for i in range(parts):
        for lo, hi in cyclic_partition_range(n, parts, i, shift):
            seen.extend(range(lo, hi))
    assert sorted(seen) == list(range(n))


@settings(max_examples=25, deadline=None)
@given(st.integers(1, 120), st.integers(0, 9), st.integers(0, 2**31 - 1))
def test_lmdb_readers_agree_on_random_environments(n, cap, seed):
    import tempfile
    from rembrandt_b200.data.lmdb_reader import LmdbEnv, NativeLmdbEnv, write_env
    rng = np.random.default_rng(seed)
    keys = sorted({bytes(rng.integers(97, 123, int(rng.integers(1, 12))).astype(np.uint8)) for _ in range(n)})
    items = [(k, bytes(rng.integers(0, 256, int(rng.choice([0, 3, 40, 700, 1500, 9000]))).astype(np.uint8))) for k in keys]
    with tempfile.TemporaryDirectory() as d:
        write_env(d, items, max_leaf_nodes=0 if cap < 3 else cap)
        probe = bytes(rng.integers(97, 123, 3).astype(np.uint8))
        with LmdbEnv(d) as a, NativeLmdbEnv(d) as b:
            assert list(a.items()) == items and list(b.items()) == items
            assert list(a.items(probe)) == list(b.items(probe)) == [kv for kv in items if kv[0] >= probe]
            assert a.get(keys[0]) == b.get(keys[0]) == items[0][1]


@settings(max_examples=40, deadline=None)
@given(st.integers(1, 5), st.integers(2, 3), st.integers(0, 2), st.integers(5, 13), st.integers(5, 13), st.integers(0, 2**31 - 1))
def test_strided_data_grad_phases_match_autograd(k, stride, pad, H, W, seed):
    import torch
    import torch.nn.functional as F
    from rembrandt_b200.ops.conv_strided import dgrad_by_phases_reference
    if pad >= k or H + 2 * pad < k or W + 2 * pad < k:
        return
    torch.manual_seed(seed)
    x = torch.randn(1, 3, H, W, dtype=torch.float64, requires_grad=True)
    w = torch.randn(4, 3, k, k, dtype=torch.float64)
    y = F.conv2d(x, w, stride=stride, padding=pad)
    dy = torch.randn_like(y)
    ref = torch.autograd.grad(y, x, dy)[0]
    got = dgrad_by_phases_reference(dy, w, H, W, stride, pad)
    assert torch.allclose(got, ref, atol=1e-9), float((got - ref).abs().max())


@settings(max_examples=120, deadline=None)
@given(st.integers(0, 4), st.integers(0, 300), st.integers(0, 300), st.binary(max_size=64), st.integers(0, 2**31 - 1),
       st.lists(st.floats(-1e3, 1e3, width=32), max_size=5), st.booleans(), st.booleans())
def test_datum_decoders_agree_on_well_formed_messages(c, h, w, data, label, floats, encoded, packed):
    from rembrandt_b200.data import codecs
    msg = codecs.encode_caffe_datum(data, c, h, w, label, encoded)
    fl = np.asarray(floats, dtype="<f4")
    if len(fl):
        if packed:
            msg += bytes([6 << 3 | 2, 4 * len(fl)]) + fl.tobytes()
        else:
            msg += b"".join(bytes([6 << 3 | 5]) + fl[i:i + 1].tobytes() for i in range(len(fl)))
    a, b = codecs.decode_caffe_datum(msg), codecs.decode_caffe_datum_py(msg)
    assert a == b
    assert a["data"] == data and a["label"] == label and a["float_data"] == fl.tolist()


@settings(max_examples=300, deadline=None)
@given(st.binary(max_size=48))
def test_native_datum_parser_never_reads_outside_arbitrary_bytes(junk):
    """Arbitrary bytes either parse (then the data field lies inside the message) or are rejected with ValueError."""
    from rembrandt_b200.data import codecs
    try:
        d = codecs.decode_caffe_datum(junk)
    except ValueError:
        return
    assert len(d["data"]) <= len(junk)


@settings(max_examples=100, deadline=None)
@given(st.integers(1, 5), st.integers(1, 9), st.integers(1, 9), st.integers(1, 255), st.integers(0, 2**31 - 1))
def test_bit_planes_round_trip(c, h, w, scale, seed):
    from rembrandt_b200.data import codecs
    bits = np.random.default_rng(seed).integers(0, 2, (c, h, w))
    out = codecs.Bits3dCodec(scale).decode(codecs.encode_bits3d(bits))
    assert out.dtype == np.uint8 and (out == bits * scale).all()
