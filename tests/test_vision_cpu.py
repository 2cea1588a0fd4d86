"""Image processor, prompt-side helpers and the tower's host metadata (CPU)."""
import base64
import io

import numpy as np
import pytest
import torch

from saber_engine_b200.vision import processor as VP
from saber_engine_b200.vision import tower as VT


def test_smart_resize_rules():
    assert VP.smart_resize(512, 512) == (512, 512)
    assert VP.smart_resize(100, 100) == (256, 256)            # lifted to the pixel floor
    h, w = VP.smart_resize(6000, 8000)
    assert h % 32 == 0 and w % 32 == 0 and h * w <= 16_777_216
    assert VP.smart_resize(48, 80, min_pixels=0) == (64, 64)   # 1.5 -> 2 and 2.5 -> 2: ties go to the even multiple
    with pytest.raises(VP.ImageInputError):
        VP.smart_resize(10, 4000)


def test_resample_matches_cpu_restatement():
    rng = np.random.default_rng(0)
    img = rng.integers(0, 256, size=(75, 131, 3), dtype=np.uint8)
    for size in [(64, 96), (160, 224)]:
        a = VP.resize(img, size).astype(np.int32)
        b = VP.resample_bicubic_aa_np(img, size).astype(np.int32)
        assert a.shape == b.shape
        assert np.abs(a - b).max() <= 2 and np.abs(a - b).mean() < 0.2


def test_patch_rows_order_and_values():
    cfg = VP.ProcessorConfig(min_pixels=0)
    rng = np.random.default_rng(1)
    img = rng.integers(0, 256, size=(64, 96, 3), dtype=np.uint8)
    out = VP.process_image(img, cfg)
    assert out.grid_thw == (1, 4, 6) and out.pixel_values.shape == (24, 1536)
    norm = img.astype(np.float32) / 255.0 * 2.0 - 1.0
    # row 5 = block (row 0, col 1) of the 2 x 3 merged grid, inner (0, 1) -> patch (0, 3)
    r = out.pixel_values[5].reshape(3, 2, 16, 16)
    want = norm[0:16, 48:64].transpose(2, 0, 1)
    assert np.allclose(r[:, 0], want, atol=1e-6) and np.array_equal(r[:, 0], r[:, 1])


def test_decode_and_data_url_round_trip():
    from PIL import Image
    img = (np.arange(40 * 50 * 3) % 251).astype(np.uint8).reshape(40, 50, 3)
    buf = io.BytesIO()
    Image.fromarray(img).save(buf, format="PNG")
    url = "data:image/png;base64," + base64.b64encode(buf.getvalue()).decode()
    back = VP.decode_image(VP.fetch_image_url(url))
    assert np.array_equal(back, img)
    with pytest.raises(VP.ImageInputError):
        VP.fetch_image_url("http://example.com/x.png")
    with pytest.raises(VP.ImageInputError):
        VP.decode_image(b"not an image")


def test_pad_expansion_and_three_axis_positions():
    PAD = 9
    grids = [(1, 4, 6)]
    ids = VP.expand_image_pads([1, 2, PAD, 3, 4], PAD, grids)
    assert ids == [1, 2] + [PAD] * 6 + [3, 4]
    pos, delta = VP.mrope_positions(ids, PAD, grids)
    assert pos[:, :2].tolist() == [[0, 1]] * 3
    assert pos[0, 2:8].tolist() == [2] * 6                      # one frame
    assert pos[1, 2:8].tolist() == [2, 2, 2, 3, 3, 3]           # merged rows
    assert pos[2, 2:8].tolist() == [2, 3, 4, 2, 3, 4]           # merged columns
    assert pos[:, 8].tolist() == [5, 5, 5] and pos[:, 9].tolist() == [6, 6, 6]
    assert delta == 7 - 10
    with pytest.raises(VP.ImageInputError):
        VP.expand_image_pads([PAD, PAD], PAD, grids)


def test_tower_metadata_shapes_and_merge_order():
    cfg = VT.VisionConfig.tiny()
    grids = [(1, 4, 6), (1, 2, 2)]
    idx, wt = VT.pos_gather_table(grids, cfg)
    assert idx.shape == (28, 4) and np.allclose(wt.sum(1), 1.0, atol=1e-5)
    assert idx.min() >= 0 and idx.max() < cfg.pos_grid ** 2
    cos, sin = VT.rope_tables(grids, cfg)
    assert cos.shape == (28, 36)
    # row 1 of the first image is patch (0, 1): row angle 0, column angle 1 * inv_freq
    assert np.allclose(sin[1, :18], 0.0) and np.isclose(sin[1, 18], np.sin(1.0))
    # row 2 is patch (1, 0) (second row of the first 2 x 2 block)
    assert np.isclose(sin[2, 0], np.sin(1.0)) and np.allclose(sin[2, 18:], 0.0)
    blocks = VT.attn_blocks([(1, 16, 16), (1, 4, 6)])
    assert blocks.tolist() == [[0, 256, 0, 0], [0, 256, 64, 0], [0, 256, 128, 0], [0, 256, 192, 0], [256, 24, 0, 0]]


def test_tower_reference_runs_and_is_image_local():
    cfg = VT.VisionConfig.tiny(depth=1, out_hidden=64)
    w = VT.VisionWeights.random(cfg, seed=3)
    g = torch.Generator().manual_seed(0)
    a = torch.randn(16, 1536, generator=g)
    b = torch.randn(24, 1536, generator=g)
    both = VT.tower_reference(cfg, w, torch.cat([a, b]), [(1, 4, 4), (1, 4, 6)])
    alone = VT.tower_reference(cfg, w, a, [(1, 4, 4)])
    assert both.shape == (10, 64)
    assert torch.allclose(both[:4], alone, atol=1e-6)           # attention never crosses images


# ------------------------------------------------------------------ image arena, request builder, scheduler plumbing
class _FakeModel:
    def __init__(self, vocab=1024, rows=64, hidden=32):
        from types import SimpleNamespace
        self.cfg = SimpleNamespace(vocab=vocab)
        self.image_rows = rows
        self.embed_table = torch.zeros(vocab + rows, hidden, dtype=torch.bfloat16)
        self.stream = None


def test_row_arena_first_fit_and_merge():
    from saber_engine_b200.vision.engine import RowArena
    a = RowArena(10)
    x, y, z = a.alloc(4), a.alloc(4), a.alloc(4)
    assert (x, y, z) == (0, 4, None)
    a.free(0, 4)
    assert a.alloc(2) == 0 and a.free_rows == 4
    a.free(4, 4)
    a.free(0, 2)
    assert a.free_rows == 10 and a.alloc(10) == 0


def test_request_builder_and_scheduler_carry_image_rows_and_positions():
    from types import SimpleNamespace
    from saber_engine_b200.sched.mock import NullExecutor
    from saber_engine_b200.sched.scheduler import Scheduler, SchedulerConfig
    from saber_engine_b200.serve.engine_api import SamplingParams
    from saber_engine_b200.vision.engine import VisionFrontend
    ex = NullExecutor(vocab=2048, max_seqs=2, prefill_rungs=(16, 64))
    ex.model = _FakeModel(vocab=1024, rows=64)
    seen = []
    pre = ex.prefill
    ex.prefill = lambda runs: (seen.extend(runs), pre(runs))[1]
    dec = ex.decode
    ex.decode = lambda runs, w: (seen.extend(runs), dec(runs, w))[1]
    calls = []

    def encode(px, grids, out_rows):
        calls.append((tuple(px.shape), list(grids)))
        out_rows.fill_(1.0)
    PAD = 300
    vis = VisionFrontend(ex, SimpleNamespace(max_patches=4096), PAD, VP.ProcessorConfig(min_pixels=0), encode=encode)
    img = np.random.default_rng(0).integers(0, 256, size=(64, 96, 3), dtype=np.uint8)
    req = vis.build_request([5, 6, PAD, 7], [img], SamplingParams(max_tokens=4, ignore_eos=True))
    assert calls == [((24, 1536), [(1, 4, 6)])]
    assert req.prompt_token_ids == [5, 6] + list(range(1024, 1030)) + [7]
    assert req.mm["rope_delta"] == -3 and vis.arena.free_rows == 58
    assert float(ex.model.embed_table[1024:1030].float().min()) == 1.0
    s = Scheduler(ex, SchedulerConfig(max_seqs=2, max_ctx=512, prefix_cache_min_tokens=4, prefix_cache_interval=4))
    sub = s.submit(req)
    s.run_until_idle()
    assert s.prefix.stats.lookups == 0 and s.prefix.stats.inserts == 0      # image rows are not content
    first = seen[0]
    assert first.rope_pos is not None and first.rope_pos[1][:5] == [0, 1, 2, 2, 2] and first.rope_pos[2][2:5] == [2, 3, 4]
    assert all(r.rope_delta == -3 for r in seen if r.rope_pos is None)
    assert vis.arena.free_rows == 64                                         # released when the request finished
    ev = sub.events.get(timeout=5)
    assert ev is not None


def test_text_only_server_refuses_image_parts():
    from saber_engine_b200.serve.server import _collect_images
    msgs = [{"role": "user", "content": [{"type": "text", "text": "hi"},
                                         {"type": "image_url", "image_url": {"url": "data:image/png;base64,AAAA"}}]}]
    with pytest.raises(ValueError):
        _collect_images(msgs, False)
    with pytest.raises(ValueError):
        _collect_images(msgs, True)              # not a decodable image
    assert _collect_images([{"role": "user", "content": "plain"}], False) == []
