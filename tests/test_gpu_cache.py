"""GPU: the on-disk cache of a built index reproduces the index bit for bit and refuses
files that do not belong to the caller's tag or are damaged."""
import os

import numpy as np
import pytest

from tests.synth import gaussian_rows

pytestmark = pytest.mark.gpu


def _rows(n, dim, seed):
    r = gaussian_rows(n, dim, seed)
    r[:, 0] += 3.0
    return r


@pytest.mark.parametrize("store,centered", [("LK_F32", True), ("LK_F32", False), ("LK_I8", False), ("LK_F16", False)])
def test_roundtrip_is_bit_identical(lk, tmp_path, store, centered):
    n, dim = 3001, 100
    idx = lk.DeviceIndex(dim, getattr(lk, store), centered=centered)
    idx.append(_rows(n, dim, 1))
    qs = _rows(5, dim, 2)
    want = idx.search(qs, 20)
    path = str(tmp_path / "media.lkidx")
    idx.save(path, tag=0xC11F0000 + n)
    back = lk.DeviceIndex.load(path, tag=0xC11F0000 + n)
    assert (len(back), back.dim, back.store, back.centered) == (n, dim, getattr(lk, store), centered)
    a, b = idx.read_rows(0, n), back.read_rows(0, n)
    if isinstance(a, tuple):
        assert all(np.array_equal(x, y) for x, y in zip(a, b))
    else:
        assert np.array_equal(a, b)
    if centered:
        sa, sb = idx.center_state(), back.center_state()
        for key in sa:
            assert np.array_equal(np.asarray(sa[key]), np.asarray(sb[key])), key
    got = back.search(qs, 20)
    for x, y in zip(want, got):
        assert np.array_equal(x, y)
    back.append(_rows(7, dim, 3))     # a loaded index keeps growing like any other
    assert len(back) == n + 7


def test_wrong_tag_truncation_and_damage_are_refused(lk, tmp_path):
    idx = lk.DeviceIndex(64, lk.LK_I8)
    idx.append(_rows(500, 64, 4))
    path = str(tmp_path / "faces.lkidx")
    idx.save(path, tag=7)
    with pytest.raises(lk.LokiError, match="another tag"):
        lk.DeviceIndex.load(path, tag=8)
    blob = open(path, "rb").read()
    open(path, "wb").write(blob[:-9])
    with pytest.raises(lk.LokiError, match="shorter"):
        lk.DeviceIndex.load(path, tag=7)
    open(path, "wb").write(blob + b"x")
    with pytest.raises(lk.LokiError, match="longer"):
        lk.DeviceIndex.load(path, tag=7)
    damaged = bytearray(blob)
    damaged[128 + 1000] ^= 0x10
    open(path, "wb").write(bytes(damaged))
    with pytest.raises(lk.LokiError, match="checksum"):
        lk.DeviceIndex.load(path, tag=7)
    open(path, "wb").write(b"not an index")
    with pytest.raises(lk.LokiError, match="not an index cache"):
        lk.DeviceIndex.load(path, tag=7)
    assert not os.path.exists(path + ".tmp")


def test_path_keyed_cache(lk, tmp_path):
    from loki_b200 import embedindex as E
    names = [f"/lib/img-{i:05d}.jpg" for i in range(800)] + ["/lib/ü ñ.png", ""]
    rows = _rows(len(names), 48, 5)
    idx = E.NewCentered()
    idx.AddBatch(names, rows)
    idx.Delete(names[3])                      # swap-remove: the cache keeps the slot order it finds
    q = rows[10]
    want = idx.Search(q, 15)
    path = str(tmp_path / "media.lkidx")
    idx.SaveCache(path, tag=len(names))
    back = E.VectorIndex.LoadCache(path, tag=len(names))
    assert back.Len() == idx.Len() == len(names) - 1
    assert [(h.Path, h.Score) for h in back.Search(q, 15)] == [(h.Path, h.Score) for h in want]
    back.Add("/lib/new.jpg", rows[0])
    assert back.Len() == len(names)
    os.remove(path + ".paths")
    with pytest.raises(E.LokiError, match="paths"):
        E.VectorIndex.LoadCache(path, tag=len(names))


def test_path_table_must_belong_to_its_rows(lk, tmp_path):
    """A path table left over from another save (same row count, same tag) or with a flipped byte is
    refused: both files must come from the same save, and the header's own fields are checksummed."""
    from loki_b200 import embedindex as E
    names = [f"/lib/{i:04d}.jpg" for i in range(300)]
    rows = _rows(300, 32, 9)
    a = E.New()
    a.AddBatch(names, rows)
    b = E.New()
    b.AddBatch(list(reversed(names)), rows)                 # same count, other path order
    pa, pb = str(tmp_path / "a.lkidx"), str(tmp_path / "b.lkidx")
    a.SaveCache(pa, tag=300)
    b.SaveCache(pb, tag=300)
    assert E.VectorIndex.LoadCache(pa, tag=300).Len() == 300
    stale = open(pb + ".paths", "rb").read()
    good = open(pa + ".paths", "rb").read()
    open(pa + ".paths", "wb").write(stale)                  # the other save's table beside these rows
    with pytest.raises(E.LokiError, match="paths"):
        E.VectorIndex.LoadCache(pa, tag=300)
    flipped = bytearray(good)
    flipped[-3] ^= 0x01                                     # one bit inside a path
    open(pa + ".paths", "wb").write(bytes(flipped))
    with pytest.raises(E.LokiError, match="paths"):
        E.VectorIndex.LoadCache(pa, tag=300)
    open(pa + ".paths", "wb").write(good)
    assert [h.Path for h in E.VectorIndex.LoadCache(pa, tag=300).Search(rows[5], 3)] == [h.Path for h in a.Search(rows[5], 3)]
    blob = bytearray(open(pa, "rb").read())
    blob[40] ^= 0x01                                        # a header field of the rows file (n_centered's neighbourhood)
    open(pa, "wb").write(bytes(blob))
    with pytest.raises(E.LokiError):
        E.VectorIndex.LoadCache(pa, tag=300)
