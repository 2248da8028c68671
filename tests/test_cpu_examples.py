"""The command-line application with the flags of the reference's applications (ResNetv1ForCifar.java:797-1029): data set
by name and directory, depth by `--layers`, training for a duration."""
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_train_py_takes_the_reference_applications_flags(tmp_path):
    from crossbow_b200.data.convert import main as convert
    d = str(tmp_path / "cifar")
    assert convert(["random", "--shape", "3,32,32", "--classes", "10", "--count", "32", "-o", d, "--name", "cifar-train", "-b", "8"]) == 0
    assert convert(["random", "--shape", "3,32,32", "--classes", "10", "--count", "16", "-o", d, "--name", "cifar-test", "-b", "8", "--seed", "3"]) == 0
    cmd = [sys.executable, os.path.join(ROOT, "examples", "train.py"), "--model", "resnet", "--layers", "8", "--dataset-name", "cifar-10",
           "--data-directory", d, "--gpu", "false", "--cpu", "true", "--number-of-cpu-models", "1", "--batch-size", "8", "--wpc", "1",
           "--update-model", "SMA", "--learning-rate", "0.01", "--time-limit", "true", "--D", "2", "--duration-unit", "seconds",
           "--display-interval", "2"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=dict(os.environ, OMP_NUM_THREADS="2"))
    assert r.returncode == 0, r.stderr[-2000:]
    shown = [l for l in r.stdout.splitlines() if l.startswith("[0") and "loss" in l]
    assert len(shown) >= 2 and "examples/s" in shown[0]
    # an invalid depth for the data set is refused the way the reference's application refuses it
    bad = subprocess.run(cmd[:5] + ["9"] + cmd[6:], capture_output=True, text=True, timeout=120)
    assert bad.returncode != 0 and "invalid number of layers" in (bad.stderr + bad.stdout)


def test_noop_application_runs_a_chain_of_copy_operators():
    """NoopApp.java / NoopStatelessApp.java: `--chain` operators that copy their input, through the whole runtime."""
    import json
    for extra in (["--chain", "4"], ["--chain", "2", "--stateless", "true"]):
        cmd = [sys.executable, os.path.join(ROOT, "examples", "noop.py"), *extra, "--N", "32", "--training-unit", "tasks", "--gpu", "false",
               "--cpu", "true", "--number-of-cpu-models", "2"]
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=dict(os.environ, OMP_NUM_THREADS="2"))
        assert r.returncode == 0, r.stderr[-2000:]
        out = json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][-1])
        assert out["tasks"] == 32 and out["tasks_per_s"] > 0 and out["chain"] == int(extra[1])
    bad = subprocess.run([sys.executable, os.path.join(ROOT, "examples", "noop.py"), "--dataset-alias", "mnist", "--gpu", "false", "--cpu", "true"],
                         capture_output=True, text=True, timeout=120)
    assert bad.returncode != 0 and "invalid dataset alias" in (bad.stderr + bad.stdout)


def test_dataset_preparation_scripts_convert_local_files(tmp_path):
    """examples/datasets/prepare-{mnist,cifar-10}.sh (the reference's scripts/datasets/*): with the original files already in
    place nothing is downloaded; the output is <data>/<set>/b-NNN/<alias>-{train,test}.metadata, readable by the data sets."""
    import struct
    import numpy as np
    g = np.random.default_rng(0)
    data = tmp_path / "data"
    orig = data / "mnist" / "original"
    orig.mkdir(parents=True)
    for prefix, n in (("train", 12), ("t10k", 6)):
        (orig / f"{prefix}-images-idx3-ubyte").write_bytes(struct.pack(">IIII", 2051, n, 28, 28) + g.integers(0, 256, n * 784, dtype=np.uint8).tobytes())
        (orig / f"{prefix}-labels-idx1-ubyte").write_bytes(struct.pack(">II", 2049, n) + g.integers(0, 10, n, dtype=np.uint8).tobytes())
    r = subprocess.run(["bash", os.path.join(ROOT, "examples", "datasets", "prepare-mnist.sh"), "4", str(data)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-1000:] + r.stderr[-2000:]
    out = data / "mnist" / "b-004"
    assert (out / "mnist-train.metadata").exists() and (out / "mnist-test.metadata").exists()
    from crossbow_b200.data.native import BasicDataset
    ds = BasicDataset(str(out / "mnist-train.metadata"), window=1)
    x, y = ds.batch(0)
    assert tuple(x.shape) == (4, 1, 28, 28) and float(x.max()) <= 1.0 and tuple(y.shape) == (4,)
    # a second run refuses to overwrite, as the reference's script does
    again = subprocess.run(["bash", os.path.join(ROOT, "examples", "datasets", "prepare-mnist.sh"), "4", str(data)], capture_output=True, text=True, timeout=120)
    assert again.returncode != 0 and "already exists" in again.stdout
    corig = data / "cifar-10" / "original"
    corig.mkdir(parents=True)
    for name, n in [(f"data_batch_{i}.bin", 4) for i in range(1, 6)] + [("test_batch.bin", 4)]:
        rec = np.concatenate([g.integers(0, 10, (n, 1), dtype=np.uint8), g.integers(0, 256, (n, 3072), dtype=np.uint8)], axis=1)
        (corig / name).write_bytes(rec.tobytes())
    r = subprocess.run(["bash", os.path.join(ROOT, "examples", "datasets", "prepare-cifar-10.sh"), "5", str(data)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-1000:] + r.stderr[-2000:]
    cout = data / "cifar-10" / "b-005"
    assert (cout / "cifar-train.metadata").exists() and (cout / "cifar-test.metadata").exists() and (cout / "cifar-train.mean").exists()
