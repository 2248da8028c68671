"""Record files, the built-in baseline JPEG decoder (against PIL / libjpeg) and the double-buffered decoding data set."""
import io

import numpy as np
import pytest

PIL = pytest.importorskip("PIL.Image")

from crossbow_b200.data.records import RecordDataset, RecordWriter, decode_jpeg, preprocess


def _image(w, h, seed=0):
    g = np.random.default_rng(seed)
    base = g.random((h // 8 + 2, w // 8 + 2, 3))
    return (np.kron(base, np.ones((8, 8, 1)))[:h, :w] * 255).astype(np.uint8)


def _jpeg(img, quality=90, subsampling=2, **kw):
    buf = io.BytesIO()
    PIL.fromarray(img).save(buf, format="JPEG", quality=quality, subsampling=subsampling, **kw)
    return buf.getvalue()


@pytest.mark.parametrize("w,h,sub", [(64, 48, 0), (67, 45, 2), (120, 90, 1), (33, 70, 2), (224, 160, 2)])
def test_decoder_matches_libjpeg(w, h, sub):
    data = _jpeg(_image(w, h), subsampling=sub)
    ref = np.array(PIL.open(io.BytesIO(data)).convert("RGB")).astype(int)
    out = decode_jpeg(data).astype(int)
    assert out.shape == ref.shape
    assert np.abs(out - ref).max() <= 2 and np.abs(out - ref).mean() < 0.1


def test_decoder_greyscale_restart_and_progressive():
    img = _image(50, 50)[..., 0]
    buf = io.BytesIO()
    PIL.fromarray(img).save(buf, format="JPEG", quality=90)
    assert np.abs(decode_jpeg(buf.getvalue())[..., 0].astype(int) - np.array(PIL.open(io.BytesIO(buf.getvalue()))).astype(int)).max() <= 1
    with pytest.raises(ValueError):
        decode_jpeg(_jpeg(_image(40, 40), progressive=True))
    with pytest.raises(ValueError):
        decode_jpeg(b"not a jpeg")


def test_test_pipeline_is_centre_crop_resize():
    img = _image(200, 120, seed=3)
    out = preprocess(_jpeg(img, quality=95, subsampling=0), training=False, size=64)
    assert out.shape == (3, 64, 64) and out.min() >= -1.0 and out.max() <= 1.0
    # reference: centred square of side round(120/1.145)=105, bilinear (corner-aligned scale) to 64
    dec = decode_jpeg(_jpeg(img, quality=95, subsampling=0)).astype(np.float32)
    cs = int(round(120 / 1.145))
    x0, y0 = (200 - cs) // 2, (120 - cs) // 2
    crop = dec[y0:y0 + cs, x0:x0 + cs]
    s = cs / 64.0
    ref = np.empty((64, 64, 3), dtype=np.float32)
    for oy in range(64):
        fy = oy * s
        iy = int(fy)
        wy = fy - iy
        iy1 = min(iy + 1, cs - 1)
        for ox in range(64):
            fx = ox * s
            ix = int(fx)
            wx = fx - ix
            ix1 = min(ix + 1, cs - 1)
            top = crop[iy, ix] + (crop[iy, ix1] - crop[iy, ix]) * wx
            bot = crop[iy1, ix] + (crop[iy1, ix1] - crop[iy1, ix]) * wx
            ref[oy, ox] = top + (bot - top) * wy
    assert np.abs(out - (ref.transpose(2, 0, 1) / 127.5 - 1)).max() < 1e-4


def test_training_pipeline_is_deterministic_per_seed_and_varies():
    data = _jpeg(_image(160, 120, seed=4))
    a = preprocess(data, boxes=[[0.2, 0.2, 0.8, 0.8]], training=True, size=32, seed=5)
    b = preprocess(data, boxes=[[0.2, 0.2, 0.8, 0.8]], training=True, size=32, seed=5)
    c = preprocess(data, boxes=[[0.2, 0.2, 0.8, 0.8]], training=True, size=32, seed=6)
    assert np.array_equal(a, b) and not np.array_equal(a, c)
    assert a.min() >= -1.0 and a.max() <= 1.0


def test_record_file_and_double_buffer(tmp_path):
    paths = []
    labels = []
    for f in range(2):
        p = str(tmp_path / f"part.{f + 1}")
        w = RecordWriter(p)
        for i in range(10):
            lab = f * 10 + i
            w.append(_jpeg(_image(48 + i, 40 + f, seed=lab)), lab, boxes=[[0.1, 0.1, 0.9, 0.9]], height=40 + f, width=48 + i)
            labels.append(lab)
        assert w.close() == 10
        paths.append(p)
    ds = RecordDataset(paths, batch_size=4, batches_per_half=2, image_size=32, workers=3, training=False, seed=1, timeout_s=20)
    assert ds.number_of_examples() == 20
    seen = []
    for b in range(10):           # 10 batches = 5 half-buffers: forces several swaps
        x, y = ds.batch(b)
        assert x.shape == (4, 3, 32, 32) and float(x.abs().max()) <= 1.0 and float(x.abs().sum()) > 0
        seen.extend(int(v) for v in y)
    assert seen[:20] == labels            # test mode keeps file order; then it wraps around
    assert seen[20:40] == labels
    assert ds.decode_failures() == 0
    # the decoded image equals the single-record pipeline
    first = preprocess(_jpeg(_image(48, 40, seed=0)), training=False, size=32)
    ds2 = RecordDataset(paths, batch_size=4, batches_per_half=2, image_size=32, workers=1, training=False, timeout_s=20)
    x, _ = ds2.batch(0)
    assert np.allclose(x[0].numpy(), first)
    ds.close()
    ds2.close()
