"""The image pre-processing kernel (crop, mirror, bilinear resize, scaling, planar layout) against the host pipeline of
the record reader: same crop plan, bit-identical examples."""
import io

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
PIL = pytest.importorskip("PIL.Image")


def _jpeg(w, h, seed, **kw):
    g = np.random.default_rng(seed)
    yy, xx = np.mgrid[0:h, 0:w]
    img = np.stack([(127 + 90 * np.sin(xx / (5.0 + c)) * np.cos(yy / (9.0 - c)) + g.normal(0, 10, (h, w))).clip(0, 255) for c in range(3)], -1).astype(np.uint8)
    buf = io.BytesIO()
    PIL.fromarray(img).save(buf, format="JPEG", quality=92, **kw)
    return buf.getvalue()


@pytest.mark.parametrize("size", [32, 224])
def test_gpu_preprocessing_is_bit_identical_to_the_host_path(size):
    from crossbow_b200.data.records import crop_plan, decode_jpeg, preprocess, preprocess_batch_gpu
    files = [_jpeg(64, 48, 1), _jpeg(333, 250, 2, progressive=True), _jpeg(500, 375, 3, subsampling=2), _jpeg(97, 211, 4), _jpeg(41, 37, 5)]
    boxes = [[[0.1, 0.2, 0.8, 0.9]], [], [[0.3, 0.3, 0.6, 0.7], [0.0, 0.0, 0.2, 0.2]], [], [[0.0, 0.0, 1.0, 1.0]]]
    for training in (True, False):
        images, plans, ref = [], [], []
        for i, (f, b) in enumerate(zip(files, boxes)):
            img = decode_jpeg(f)
            images.append(img)
            plans.append(crop_plan(img.shape[1], img.shape[0], b, training, seed=100 + i))
            ref.append(preprocess(f, b, training, size, seed=100 + i))
        out = preprocess_batch_gpu(images, plans, size)
        torch.cuda.synchronize()
        got = out.cpu().numpy()
        assert got.shape == (len(files), 3, size, size)
        for i in range(len(files)):
            assert np.array_equal(got[i], ref[i]), (training, i, float(np.abs(got[i] - ref[i]).max()))
        assert got.min() >= -1.0 and got.max() <= 1.0


def test_gpu_preprocessing_rejects_a_window_outside_the_image():
    from crossbow_b200.data.records import preprocess_batch_gpu
    img = np.zeros((20, 30, 3), dtype=np.uint8)
    with pytest.raises(ValueError):
        preprocess_batch_gpu([img], [(10, 5, 25, 10, 0)], 16)
