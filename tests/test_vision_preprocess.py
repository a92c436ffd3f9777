"""Image preprocessing: the resize rule, byte-exactness of the bicubic against PIL, patch order and position ids."""
import numpy as np
import pytest

from rexl3_b200 import vision


def test_smart_resize_rule():
    h, w = vision.smart_resize(1080, 1920)
    assert h % 28 == 0 and w % 28 == 0
    assert h * w <= 14 * 14 * 4 * 1280 and abs(h / w - 1080 / 1920) < 0.02
    h, w = vision.smart_resize(20, 30)
    assert h % 28 == 0 and w % 28 == 0 and h * w >= 56 * 56
    assert vision.smart_resize(280, 280) == (280, 280)
    with pytest.raises(ValueError):
        vision.smart_resize(10, 5000)


@pytest.mark.parametrize("shape,out", [((37, 53), (56, 84)), ((200, 120), (56, 28)), ((64, 64), (64, 140)), ((90, 160), (90, 160)), ((300, 7), (28, 28))])
def test_bicubic_is_byte_exact_with_pil(shape, out):
    Image = pytest.importorskip("PIL.Image")
    rng = np.random.default_rng(shape[0] * 1000 + out[1])
    img = rng.integers(0, 256, size=shape + (3,), dtype=np.uint8)
    img[: shape[0] // 3] = np.clip(img[: shape[0] // 3].astype(int) // 8 * 8, 0, 255)       # flat-ish band
    want = np.asarray(Image.fromarray(img).resize((out[1], out[0]), Image.BICUBIC))
    got = vision.bicubic_resize_u8(img, out[0], out[1])
    assert got.shape == want.shape and np.array_equal(got, want)


def test_patch_order_and_position_ids():
    t, c, h, w, p, m = 1, 3, 56, 84, 14, 2
    frames = np.arange(t * c * h * w, dtype=np.float32).reshape(t, c, h, w)
    rows, grid = vision.patchify(frames, p, m, 2)
    assert grid == (1, 4, 6) and rows.shape == (24, 3 * 2 * 14 * 14)
    ids = vision.patch_position_ids(grid, m)
    assert ids.shape == (24, 2)
    # the first four rows are the 2x2 block the merger fuses: tiles (0,0), (0,1), (1,0), (1,1)
    assert ids[:4].tolist() == [[0, 0], [0, 1], [1, 0], [1, 1]] and ids[4].tolist() == [0, 2]
    for r in (0, 3, 5, 17):
        gh, gw = ids[r]
        tile = frames[0, :, gh * p:(gh + 1) * p, gw * p:(gw + 1) * p]                        # [c, p, p]
        want = np.stack([tile, tile], axis=1).reshape(-1)                                    # the single frame repeated to the temporal patch
        assert np.array_equal(rows[r], want)


def test_preprocess_image_end_to_end():
    rng = np.random.default_rng(3)
    img = rng.integers(0, 256, size=(100, 150, 4), dtype=np.uint8)
    out = vision.preprocess_image(img)
    gt, gh, gw = out.grid_thw
    assert gt == 1 and gh % 2 == 0 and gw % 2 == 0 and out.pixel_values.shape == (gh * gw, 3 * 2 * 14 * 14)
    assert out.image_tokens == gh * gw // 4 and out.position_ids.max(axis=0).tolist() == [gh - 1, gw - 1]
    assert out.pixel_values.dtype == np.float32 and np.isfinite(out.pixel_values).all()
    lo, hi = (0 - 0.48145466) / 0.26862954, (1 - 0.40821073) / 0.27577711
    assert out.pixel_values.min() >= lo - 1e-4 and out.pixel_values.max() <= hi + 1e-4


def test_preprocess_video_pairs_frames():
    rng = np.random.default_rng(4)
    frames = [rng.integers(0, 256, size=(60, 90, 3), dtype=np.uint8) for _ in range(5)]
    out = vision.preprocess_video(frames)
    gt, gh, gw = out.grid_thw
    assert gt == 3 and out.pixel_values.shape == (3 * gh * gw, 3 * 2 * 14 * 14)          # five frames -> three pairs (the last frame repeated)
    one = vision.preprocess_image(frames[0], max_pixels=14 * 14 * 4 * 320)
    assert one.grid_thw[1:] == (gh, gw)
    # the first temporal patch holds frames 0 and 1: its first half equals the single-image rows' first half
    a = out.pixel_values[0].reshape(3, 2, 14, 14)
    b = one.pixel_values[0].reshape(3, 2, 14, 14)
    assert np.array_equal(a[:, 0], b[:, 0]) and not np.array_equal(a[:, 1], b[:, 1])
    assert out.position_ids.shape == (3 * gh * gw, 2) and np.array_equal(out.position_ids[:gh * gw], out.position_ids[gh * gw:2 * gh * gw])
    with pytest.raises(ValueError):
        vision.preprocess_video([frames[0], frames[1][:30]])
