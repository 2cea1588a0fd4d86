"""Host-side native code: streaming loader, CPU twin, ShmLine (no GPU needed)."""
import os
import threading

import numpy as np
import pytest

from saber_engine_b200.ops import cpux
from saber_engine_b200.pack import format as PF
from saber_engine_b200.pack.stream import PackStream
from saber_engine_b200.parallel.shmline import ShmLine, TornRead


def test_stream_loader_verifies_chunks(tmp_path):
    w = PF.PackWriter(tmp_path / "rank0.pack", 1, 0, {"p": 1}, {"t": 1}, build_unix=0)
    big = np.random.default_rng(0).integers(0, 255, 9 << 20, dtype=np.uint8)     # three 4 MiB chunks
    w.add("big", big, "u8")
    w.add("small", np.arange(100, dtype=np.float32), "f32")
    w.finish()
    s = PackStream(tmp_path / "rank0.pack")
    assert np.array_equal(s.read_host("big"), big)
    assert np.array_equal(s.read_host("small").view(np.float32), np.arange(100, dtype=np.float32))
    assert s.stats["chunks_verified"] == 4 and s.stats["bytes"] == big.size + 400
    s.close()
    # corrupt one byte of the second chunk: the loader names the chunk and stops
    raw = bytearray((tmp_path / "rank0.pack").read_bytes())
    off = PF.PackReader(tmp_path / "rank0.pack").records["big"].data_off + (5 << 20)
    raw[off] ^= 1
    (tmp_path / "rank0.pack").write_bytes(bytes(raw))
    s = PackStream(tmp_path / "rank0.pack")
    with pytest.raises(PF.PackError, match="chunk 1"):
        s.read_host("big")
    s.read_host("small")
    s.close()


def test_cpu_twin_simd_equals_scalar_law_and_reference():
    rng = np.random.default_rng(1)
    M, N, K = 5, 48, 256
    wq = rng.integers(-8, 8, (N, K)).astype(np.int8)
    ws = rng.random(N).astype(np.float32) * 0.01
    x = rng.standard_normal((M, K)).astype(np.float32)
    aq, asc = cpux.quant_rows(x)
    nib = cpux.pack_nibbles(wq)
    a = cpux.gemm_w4a8(aq, asc, nib, ws, simd=True)
    b = cpux.gemm_w4a8(aq, asc, nib, ws, simd=False)
    assert a.tobytes() == b.tobytes()                         # byte-equal twin
    ref = (aq.astype(np.int64) @ wq.astype(np.int64).T).astype(np.float32) * (asc[:, None] * ws[None, :])
    assert np.allclose(a, ref, rtol=1e-2, atol=1e-6)
    # control that must fail: a nibble-swapped pack is NOT equal
    swapped = ((nib << 4) | (nib >> 4)).astype(np.uint8)
    assert cpux.gemm_w4a8(aq, asc, swapped, ws).tobytes() != a.tobytes()
    # expert chain: simd == scalar, finite, right shape
    H, I = 256, 128
    wgu = cpux.pack_nibbles(rng.integers(-8, 8, (2 * I, H)).astype(np.int8))
    wd = cpux.pack_nibbles(rng.integers(-8, 8, (H, I)).astype(np.int8))
    sgu, sd = np.full(2 * I, 0.01, np.float32), np.full(H, 0.01, np.float32)
    xe = rng.standard_normal((3, H)).astype(np.float32)
    o1 = cpux.expert_chain(xe, wgu, sgu, wd, sd, simd=True)
    o2 = cpux.expert_chain(xe, wgu, sgu, wd, sd, simd=False)
    assert o1.shape == (3, H) and o1.tobytes() == o2.tobytes() and np.isfinite(o1).all()


def test_shmline_frames_and_torn_read_control():
    name = f"/saber-test-{os.getpid()}"
    w = ShmLine(name, create=True)
    r = ShmLine(name, create=False)
    got = []
    t = threading.Thread(target=lambda: got.extend(r.take(i, 2.0) for i in range(50)))
    t.start()
    for i in range(50):
        while True:
            try:
                w.post(f"frame-{i}".encode())
                break
            except BlockingIOError:          # both slots still unread: the checked post refuses to lap
                pass
    t.join()
    assert got == [f"frame-{i}".encode() for i in range(50)]
    with pytest.raises(TimeoutError):
        r.take(50, 0.05)
    r.close()
    w.close()
    # the hazard, reproduced deterministically: ONE slot and unchecked posts overwrite an unread frame
    name2 = name + "-ctl"
    w = ShmLine(name2, create=True, one_slot_control=True)
    r = ShmLine(name2, create=False, one_slot_control=True)
    w.post(b"first", checked=False)
    w.post(b"second", checked=False)
    with pytest.raises(TornRead):
        r.take(0, 0.1)
    r.close()
    w.close()
