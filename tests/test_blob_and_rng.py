"""NdArray blob codec (byte-exact), xorshift128+ streams and partition helpers (CPU)."""
import struct

import numpy as np
import pytest

from rembrandt_b200.utils import blob
from rembrandt_b200.utils.rng import XorShift128Plus, cyclic_partition_range, partition_range


def test_record_layout_is_byte_exact():
    data = np.arange(6, dtype=np.float32)
    rec = blob.encode_record(data, (3, 2))
    expect = b"ND\x00\x01" + struct.pack("<I", 2) + struct.pack("<QQ", 3, 2) + data.tobytes()
    assert rec == expect
    recs, off = blob.decode_records(rec)
    assert off == len(rec)
    arr, dims, tag = recs[0]
    assert dims == (3, 2) and tag == (0, 1) and np.array_equal(arr, data)


def test_tag_bytes_are_preserved_and_rewritten():
    rec = bytearray(blob.encode_record(np.zeros(4, np.float32), (4,)))
    rec[2], rec[3] = 0x7F, 0x03
    (arr, dims, tag), = blob.decode_records(bytes(rec))[0]
    assert tag == (0x7F, 0x03)
    assert blob.encode_record(arr, dims, tag=tag) == bytes(rec)


def test_concatenated_records_and_u8():
    a = blob.encode_record(np.arange(12, dtype=np.uint8), (2, 3, 2), dtype="u8")
    b = blob.encode_record(np.ones(5, np.float32), (1, 5))
    recs, off = blob.decode_records(a, "u8")
    assert recs[0][1] == (2, 3, 2) and off == len(a)
    both, _ = blob.decode_records(blob.encode_many([(np.ones(2), (2, 1)), (np.zeros(3), (1, 3))]))
    assert [r[1] for r in both] == [(2, 1), (1, 3)]
    assert len(b) == 8 + 16 + 20


@pytest.mark.parametrize("mutate,msg", [(lambda r: r[:6], "truncated header"), (lambda r: b"XX" + r[2:], "bad magic"),
                                        (lambda r: r[:-3], "truncated data")])
def test_corrupt_blobs_are_rejected(mutate, msg):
    rec = blob.encode_record(np.arange(8, dtype=np.float32), (8, 1))
    with pytest.raises(blob.BlobError, match=msg):
        blob.decode_records(mutate(rec))


def test_array_file_round_trip(tmp_path):
    mean = np.random.default_rng(0).random((3, 4, 5)).astype(np.float32)   # [c][h][w]
    p = tmp_path / "mean.ndarray"
    blob.write_array_file(str(p), mean)
    raw = p.read_bytes()
    assert struct.unpack("<QQQ", raw[8:32]) == (5, 4, 3)                     # dims stored as (w, h, c)
    assert np.array_equal(blob.read_array_file(str(p)), mean)


def test_xorshift_is_deterministic_and_seed_sensitive():
    a, b, c = XorShift128Plus(1, 2), XorShift128Plus(1, 2), XorShift128Plus(1, 3)
    sa = [a.next_u64() for _ in range(5)]
    assert sa == [b.next_u64() for _ in range(5)]
    assert sa != [c.next_u64() for _ in range(5)]
    # first output of xorshift128+ from state (1, 2): s1 = 1 ^ (1 << 23); new s[1] = s1 ^ 2 ^ (s1 >> 17) ^ (2 >> 26)
    s1 = 1 ^ (1 << 23)
    expect = ((s1 ^ 2 ^ (s1 >> 17) ^ (2 >> 26)) + 2) & (2**64 - 1)
    assert sa[0] == expect


def test_draws_have_the_right_moments():
    r = XorShift128Plus(5, 6)
    u = r.uniform(20000, -0.5, 0.5).numpy()
    n = r.normal(20000, 1.0, 2.0).numpy()
    assert abs(u.mean()) < 0.01 and abs(u.std() - (1 / 12) ** 0.5) < 0.01 and u.min() >= -0.5 and u.max() < 0.5
    assert abs(n.mean() - 1.0) < 0.05 and abs(n.std() - 2.0) < 0.05
    p = r.permutation(17)
    assert sorted(p) == list(range(17))
    assert all(0 <= r.below(7) < 7 for _ in range(100))


def test_derived_streams_differ_but_are_reproducible():
    root1, root2 = XorShift128Plus(9, 9), XorShift128Plus(9, 9)
    a1, b1 = root1.derive(), root1.derive()
    a2 = root2.derive()
    assert a1.next_u64() == a2.next_u64()
    assert a1.next_u64() != b1.next_u64()


def test_partition_range_is_balanced_and_covers():
    for n, parts in ((10, 3), (7, 7), (5, 8), (100, 6)):
        bounds = [partition_range(n, parts, i) for i in range(parts)]
        assert bounds[0][0] == 0 and bounds[-1][1] == n
        assert all(bounds[i][1] == bounds[i + 1][0] for i in range(parts - 1))
        sizes = [b - a for a, b in bounds]
        assert max(sizes) - min(sizes) <= 1


def test_cyclic_partition_wraps():
    pieces = cyclic_partition_range(10, 2, 1, 7)      # part [5,10) shifted by 7 -> [2,7)
    assert pieces == [(2, 7)]
    pieces = cyclic_partition_range(10, 2, 0, 7)      # part [0,5) shifted by 7 -> [7,10) + [0,2)
    assert pieces == [(7, 10), (0, 2)]
