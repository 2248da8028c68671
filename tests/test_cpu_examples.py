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
