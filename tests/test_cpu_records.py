"""Record files, the built-in JPEG decoder (sequential, progressive, CMYK; against PIL / libjpeg) and the double-buffered
decoding data set."""
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


def test_decoder_greyscale_and_garbage():
    img = _image(50, 50)[..., 0]
    buf = io.BytesIO()
    PIL.fromarray(img).save(buf, format="JPEG", quality=90)
    assert np.abs(decode_jpeg(buf.getvalue())[..., 0].astype(int) - np.array(PIL.open(io.BytesIO(buf.getvalue()))).astype(int)).max() <= 1
    with pytest.raises(ValueError):
        decode_jpeg(b"not a jpeg")


@pytest.mark.parametrize("w,h,sub,q", [(40, 40, 2, 90), (67, 45, 2, 75), (120, 90, 1, 95), (64, 48, 0, 50), (33, 70, 2, 85)])
def test_progressive_matches_libjpeg(w, h, sub, q):
    """Progressive files (spectral selection + successive approximation, separate DC / AC scans per component)."""
    data = _jpeg(_image(w, h, seed=w), quality=q, subsampling=sub, progressive=True)
    assert b"\xff\xc2" in data                       # really a progressive frame
    ref = np.array(PIL.open(io.BytesIO(data)).convert("RGB")).astype(int)
    out = decode_jpeg(data).astype(int)
    assert out.shape == ref.shape
    assert np.abs(out - ref).max() <= 2 and np.abs(out - ref).mean() < 0.1


def test_progressive_greyscale_and_natural_content():
    g = np.random.default_rng(5)
    yy, xx = np.mgrid[0:96, 0:80]
    img = (127 + 80 * np.sin(xx / 7.0) * np.cos(yy / 11.0) + g.normal(0, 12, (96, 80))).clip(0, 255).astype(np.uint8)
    for mode in ("L", "RGB"):
        im = PIL.fromarray(img) if mode == "L" else PIL.fromarray(np.stack([img, img[::-1], img[:, ::-1]], -1))
        buf = io.BytesIO()
        im.save(buf, format="JPEG", quality=88, progressive=True)
        ref = np.array(PIL.open(io.BytesIO(buf.getvalue())).convert("RGB")).astype(int)
        out = decode_jpeg(buf.getvalue()).astype(int)
        assert np.abs(out - ref).max() <= 3 and np.abs(out - ref).mean() < 0.15


def test_cmyk_files_are_converted_like_the_reference():
    """Four-component files: Adobe CMYK / YCCK (inks stored inverted), r = k * c / 255 as image/image.c:119-139 does."""
    rgb = _image(48, 40, seed=9)
    cmyk = PIL.fromarray(rgb).convert("CMYK")
    for progressive in (False, True):
        buf = io.BytesIO()
        cmyk.save(buf, format="JPEG", quality=95, subsampling=0, progressive=progressive)
        dec = PIL.open(io.BytesIO(buf.getvalue()))
        assert dec.mode == "CMYK"
        raw = np.array(dec).astype(int)               # PIL hands out the inks non-inverted
        inv = 255 - raw                               # ... libjpeg itself hands out Adobe files inverted
        ref = (inv[..., 3:4] * inv[..., :3]) // 255
        out = decode_jpeg(buf.getvalue()).astype(int)
        assert out.shape == ref.shape and np.abs(out - ref).max() <= 3


def test_restart_intervals():
    img = _image(96, 64, seed=4)
    buf = io.BytesIO()
    PIL.fromarray(img).save(buf, format="JPEG", quality=90, subsampling=2, restart_marker_blocks=3)
    data = buf.getvalue()
    if b"\xff\xdd" not in data:
        pytest.skip("this PIL build does not write restart intervals")
    ref = np.array(PIL.open(io.BytesIO(data)).convert("RGB")).astype(int)
    assert np.abs(decode_jpeg(data).astype(int) - ref).max() <= 2


def test_malformed_files_fail_cleanly():
    """Untrusted input: truncations and corrupted table selectors / lengths end in an error or a partial image, never in
    an out-of-range access (the self-test binary runs the same cases under AddressSanitizer)."""
    good = _jpeg(_image(64, 48), subsampling=2)
    prog = _jpeg(_image(64, 48), subsampling=2, progressive=True)
    for data in (good, prog):
        for cut in (3, 20, 100, len(data) // 2, len(data) - 2):
            try:
                out = decode_jpeg(data[:cut])
                assert out.shape == (48, 64, 3)       # a truncated scan keeps what was decoded
            except ValueError:
                pass
        sos = data.index(b"\xff\xda")
        for off, val in ((5, 0x7F), (6, 0xFF), (4, 9), (2, 0), (3, 1)):   # component selector, table ids, count, length
            bad = bytearray(data)
            bad[sos + off] = val
            try:
                decode_jpeg(bytes(bad))
            except ValueError:
                pass
        dht = data.index(b"\xff\xc4")
        for off in range(4, 24, 3):
            bad = bytearray(data)
            bad[dht + off] = 0xFF
            try:
                decode_jpeg(bytes(bad))
            except ValueError:
                pass
        dqt = data.index(b"\xff\xdb")
        bad = bytearray(data)
        bad[dqt + 4] = 0x10                           # claims 16-bit entries in a segment sized for 8-bit ones
        try:
            decode_jpeg(bytes(bad))
        except ValueError:
            pass
    g = np.random.default_rng(0)
    for _ in range(200):                              # random byte flips anywhere behind the SOI
        bad = bytearray(good if g.random() < 0.5 else prog)
        for _ in range(int(g.integers(1, 6))):
            bad[int(g.integers(2, len(bad)))] = int(g.integers(0, 256))
        try:
            decode_jpeg(bytes(bad))
        except ValueError:
            pass


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


def test_crop_plan_follows_the_reference_sampler():
    """Training crops: aspect ratio in [0.75, 1.33], area in [5 %, 100 %] of the image, inside the image, covering part of a
    labelled box; heights are spread over the whole admissible range (the reference draws the HEIGHT uniformly,
    image/image.c:838-860).  Test crops: the centred square of side min(W, H) / 1.145."""
    from crossbow_b200.data.records import crop_plan
    W, H = 320, 240
    hs, flips = [], 0
    for seed in range(400):
        x0, y0, cw, ch, flip = crop_plan(W, H, [[0.25, 0.25, 0.75, 0.75]], True, seed)
        assert 0 <= x0 and 0 <= y0 and x0 + cw <= W and y0 + ch <= H and cw >= 1 and ch >= 1
        if (cw, ch) != (W, H):
            assert 0.05 * W * H - 1 <= cw * ch <= W * H and 0.74 <= cw / ch <= 1.35
            ix = max(0, min(x0 + cw, 240) - max(x0, 80)); iy = max(0, min(y0 + ch, 180) - max(y0, 60))
            assert ix * iy / (cw * ch) >= 0.1
        hs.append(ch)
        flips += flip
    assert min(hs) < 0.45 * H and max(hs) > 0.9 * H and 120 < flips < 280
    assert crop_plan(W, H, [], False, 0) == ((W - 210) // 2, (H - 210) // 2, 210, 210, 0)
    assert crop_plan(W, H, [], True, 5) == crop_plan(W, H, [], True, 5)           # a function of the seed


def test_tfrecord_files_become_record_files(tmp_path):
    """ImageNet TFRecords -> record files without TensorFlow: the container's checksums, the three protobuf messages of an
    Example (packed and one-field-per-value lists), labels moved to 0..999, boxes kept, files rotated by record count."""
    import struct
    from crossbow_b200.data import tfrecords as T
    assert T.crc32c(b"123456789") == 0xE3069283
    examples, labels = [], []
    for i in range(5):
        lab = 1 + 37 * i
        examples.append(T.make_example({"image/encoded": [_jpeg(_image(40 + i, 36, seed=i))], "image/class/label": [lab],
                                        "image/height": [36], "image/width": [40 + i], "image/class/text": [b"n0%d" % i],
                                        "image/object/bbox/xmin": [0.1, 0.2][:1 + i % 2], "image/object/bbox/ymin": [0.1, 0.2][:1 + i % 2],
                                        "image/object/bbox/xmax": [0.9, 0.8][:1 + i % 2], "image/object/bbox/ymax": [0.9, 0.8][:1 + i % 2]}))
        labels.append(lab - 1)
    src = [str(tmp_path / "train-00000-of-00002"), str(tmp_path / "train-00001-of-00002")]
    assert T.write_tfrecord(src[0], examples[:3]) == 3 and T.write_tfrecord(src[1], examples[3:]) == 2
    ex = T.parse_example(next(T.read_tfrecord(src[0], verify=True)))
    assert ex["image/class/label"] == [1] and ex["image/width"] == [40] and ex["image/class/text"] == [b"n00"]
    assert ex["image/object/bbox/xmin"] == pytest.approx([0.1]) and decode_jpeg(ex["image/encoded"][0]).shape == (36, 40, 3)
    # lists written one value per field (the unpacked form older writers emit) and negative integers
    unpacked = T._ld(1, T._ld(1, T._ld(1, b"k") + T._ld(2, T._ld(3, T._put_varint(1 << 3) + T._put_varint(-5) + T._put_varint(1 << 3) + T._put_varint(7))))
                        + T._ld(1, T._ld(1, b"f") + T._ld(2, T._ld(2, bytes([1 << 3 | 5]) + struct.pack("<f", 0.25)))))
    assert T.parse_example(unpacked) == {"k": [-5, 7], "f": [0.25]}
    for cut in (1, 3, len(unpacked) - 2):                       # truncated messages are refused, not misread
        with pytest.raises(ValueError):
            T.parse_example(unpacked[:cut])
    out = T.convert_imagenet([str(tmp_path / "train-*-of-*")], str(tmp_path / "out"), "train", max_records_per_file=2, verify=True)
    assert [p.rsplit("/", 1)[1] for p in out] == ["crossbow-train.records.1", "crossbow-train.records.2", "crossbow-train.records.3"]
    ds = RecordDataset(out, batch_size=5, batches_per_half=1, image_size=32, workers=2, training=False, timeout_s=20)
    assert ds.number_of_examples() == 5
    x, y = ds.batch(0)
    assert [int(v) for v in y] == labels and ds.decode_failures() == 0
    assert np.allclose(x[0].numpy(), preprocess(_jpeg(_image(40, 36, seed=0)), training=False, size=32))
    ds.close()
    # damage: a flipped payload byte is caught by verify, a flipped length byte always
    raw = bytearray(open(src[1], "rb").read())
    raw[40] ^= 0xFF
    open(src[1], "wb").write(bytes(raw))
    with pytest.raises(ValueError, match="checksum"):
        list(T.read_tfrecord(src[1], verify=True))
    raw[40] ^= 0xFF
    raw[2] ^= 0x01
    open(src[1], "wb").write(bytes(raw))
    with pytest.raises(ValueError, match="length"):
        list(T.read_tfrecord(src[1]))
