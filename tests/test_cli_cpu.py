"""The command-line entry points run end to end on CPU with tiny settings."""
import os

import pytest

from rembrandt_b200.cli import (bench_kernels, dist_train_mnist, run_rembrandt, test_dist, train_cifar10, train_gogod,
                                train_mnist)

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TINY = ["--device", "cpu", "--batch", "8", "--iters", "3", "--display-iters", "1", "--synthetic-size", "64"]


def test_train_mnist_and_its_distributed_alias():
    sgd = train_mnist.main(TINY + ["--valid-iters", "0"])
    assert sgd.engine.iter == 3
    assert dist_train_mnist.main(TINY + ["--valid-iters", "0", "--model", "fc1"]).engine.iter == 3


def test_train_cifar10():
    assert train_cifar10.main(TINY).engine.iter == 3


@pytest.mark.parametrize("arch", ["resnet", "plain"])
def test_train_gogod(arch):
    sgd = train_gogod.main(TINY + ["--arch", arch, "--channels", "8", "--blocks", "2", "--planes", "6"])
    assert sgd.engine.iter == 3
    assert sgd.engine.net.loss_op.k == 361


def test_run_rembrandt_from_descriptors():
    sgd = run_rembrandt.main(TINY + ["--model-file", os.path.join(ROOT, "examples", "mnist_lenet.model"),
                                     "--data", os.path.join(ROOT, "examples", "synthetic_mnist.data"),
                                     "--valid-iters", "1"])
    assert sgd.engine.iter == 3


def test_host_side_probes():
    res = bench_kernels.main(["--no-device"])
    assert [r["requested_us"] for r in res["sleep"]] == [1, 10, 100, 1000, 10000]
    assert all(r["observed_us"] >= r["requested_us"] for r in res["sleep"])
    assert test_dist.main(["--device", "cpu"]) == (0, 1)


def test_training_from_a_caffe_database_through_the_native_loader(tmp_path):
    import numpy as np
    from rembrandt_b200.data.codecs import encode_caffe_datum
    from rembrandt_b200.data.lmdb_reader import write_env
    rng = np.random.default_rng(0)
    items = [(b"%08d" % i, encode_caffe_datum(rng.integers(0, 256, 3 * 32 * 32, dtype=np.uint8).tobytes(), 3, 32, 32,
                                              label=i % 10)) for i in range(64)]
    (tmp_path / "db").mkdir()
    write_env(str(tmp_path / "db"), items)
    (tmp_path / "c.data").write_text(f'[dataset.train]\nsource = "lmdb_caffe"\ndata_path = "{tmp_path / "db"}"\n')
    sgd = train_cifar10.main(TINY + ["--data", str(tmp_path / "c.data"), "--native-loader", "2"])
    assert sgd.engine.iter == 3


@pytest.mark.parametrize("comm", ["allreduce", "gossip_pair", "gossip_pull", "gossip_push", "group_allreduce_gossip", "elastic",
                                  "gossip_push_async", "elastic_async"])
def test_distributed_tool_on_two_cpu_ranks(comm):
    import socket
    import subprocess
    import sys
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), "-m", "rembrandt_b200.cli.dist_train_mnist", *TINY, "--model", "fc1",
           "--comm", comm, "--iters", "4", "--display-iters", "2", "--valid-iters", "0"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert "iter 4 " in r.stderr


def test_ranks_started_by_hand_meet_through_a_shared_directory(tmp_path):
    """No launcher: every rank is its own command with --rendezvous-dir / --rank / --world-size; a training tool
    takes the same flags."""
    import subprocess
    import sys
    env = {k: v for k, v in os.environ.items() if k not in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_ADDR", "MASTER_PORT")}

    def start(module, extra, d):
        return [subprocess.Popen([sys.executable, "-m", module, "--device", "cpu", "--rendezvous-dir", d,
                                  "--rank", str(r), "--world-size", "2", *extra], cwd=ROOT, env=env,
                                 stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True) for r in range(2)]
    outs = [p.communicate(timeout=240) + (p.returncode,) for p in start("rembrandt_b200.cli.test_dist", [], str(tmp_path / "a"))]
    assert all(rc == 0 for _, _, rc in outs), outs
    assert sorted(o.strip().splitlines()[-1][:11] for o, _, _ in outs) == ["rank 0 of 2", "rank 1 of 2"]
    tiny = [a for a in TINY if a not in ("--device", "cpu")]
    outs = [p.communicate(timeout=300) + (p.returncode,)
            for p in start("rembrandt_b200.cli.dist_train_mnist",
                           [*tiny, "--model", "fc1", "--comm", "gossip_pair", "--iters", "4", "--display-iters", "2",
                            "--valid-iters", "0"], str(tmp_path / "b"))]
    assert all(rc == 0 for _, _, rc in outs), [e[-3000:] for _, e, _ in outs]
    assert any("iter 4 " in e for _, e, _ in outs)                      # rank 0 prints the progress lines


def test_straggler_tool_on_three_cpu_ranks_shows_who_waits():
    """Lock-step push gossip: everybody pays the sleeping rank's delay. Asynchronous: only the sleeper does."""
    import json
    import socket
    import subprocess
    import sys
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=3", "--master-addr", "127.0.0.1",
           "--master-port", str(port), "-m", "rembrandt_b200.cli.bench_straggler", "--device", "cpu", "--batch", "8",
           "--comm", "gossip_push", "--both", "--delay-ms", "60", "--steps", "8", "--warmup", "2"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=400, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    rows = [json.loads(l) for l in r.stdout.splitlines() if l.startswith("{")]
    by = {(row["synchronous"], row["delay_ms"] > 0): row for row in rows}
    assert len(by) == 4
    lock, free = by[(True, True)], by[(False, True)]
    assert min(lock["ms_per_step_by_rank"]) >= 60.0                       # every rank waits for the sleeper
    assert free["ms_per_step_by_rank"][1] >= 60.0                         # the sleeper itself
    assert free["ms_per_step_of_the_other_ranks"] < lock["ms_per_step_of_the_other_ranks"] - 30.0


def test_variable_size_template_through_the_imagenet_tool(monkeypatch):
    from rembrandt_b200.cli import train_imagenet
    from rembrandt_b200.models import zoo
    full = zoo.resnet18_var
    monkeypatch.setattr(zoo, "resnet18_var", lambda: full(num_classes=10, in_hw=32, scale=(36, 40), max_hw=48))
    sgd = train_imagenet.main(["--device", "cpu", "--batch", "2", "--iters", "2", "--display-iters", "1",
                               "--synthetic-size", "8", "--model", "resnet18_var"])
    assert sgd.engine.iter == 2


def test_tool_resumes_from_the_latest_state_or_a_given_iteration(tmp_path):
    d = str(tmp_path / "run")
    args = TINY + ["--valid-iters", "0", "--model", "fc1", "--checkpoint-dir", d, "--checkpoint-iters", "2"]
    first = train_mnist.main(args + ["--iters", "4"])
    assert first.engine.iter == 4 and os.path.exists(os.path.join(d, "params.t_4.blob"))
    again = train_mnist.main(args + ["--iters", "6"])                      # picks up at 4
    rows = open(os.path.join(d, "trace_sgd.0.log.1")).read().splitlines()
    assert again.engine.iter == 6 and [r.split(",")[0] for r in rows[1:] if ",step," in r] == ["5", "6"]
    from_two = train_mnist.main(args + ["--iters", "3", "--resume-from", "2"])
    rows = open(os.path.join(d, "trace_sgd.0.log.2")).read().splitlines()
    assert from_two.engine.iter == 3 and [r.split(",")[0] for r in rows[1:] if ",step," in r] == ["3"]


@pytest.mark.parametrize("tool", ["train_mnist", "dist_train_mnist", "train_cifar10", "train_imagenet",
                                  "dist_train_imagenet", "train_gogod", "run_rembrandt", "bench_conv", "bench_gemm",
                                  "bench_allreduce", "bench_link", "bench_kernels", "bench_ops", "bench_straggler", "bench_loader", "data_tools",
                                  "test_dist"])
def test_every_tool_imports_and_prints_its_help(tool, capsys):
    import importlib
    mod = importlib.import_module(f"rembrandt_b200.cli.{tool}")
    with pytest.raises(SystemExit) as e:
        mod.main(["--help"])
    assert e.value.code == 0 and "usage:" in capsys.readouterr().out


def test_run_rembrandt_takes_optimizer_defaults_from_the_model_file():
    sgd = run_rembrandt.main(["--device", "cpu", "--batch", "16", "--iters", "2", "--display-iters", "1",
                              "--synthetic-size", "64", "--valid-iters", "0",
                              "--model-file", os.path.join(ROOT, "examples", "cifar10_krizh26.model"),
                              "--data", os.path.join(ROOT, "examples", "synthetic_cifar10.data")])
    assert sgd.cfg.minibatch_size == 128 and sgd.cfg.mu == 0.9 and sgd.cfg.l2_reg_coef == 5e-4
    assert sgd.engine.accum == 8 and sgd.engine.iter == 2
    assert sgd.cfg.step_size.at_iter(0) == 0.01 and abs(sgd.cfg.step_size.at_iter(60000) - 1e-4) < 1e-12
    # a flag on the command line wins over the file
    sgd = run_rembrandt.main(["--device", "cpu", "--batch", "8", "--minibatch", "8", "--iters", "1", "--display-iters", "1",
                              "--synthetic-size", "64", "--valid-iters", "0", "--l2", "0.0",
                              "--model-file", os.path.join(ROOT, "examples", "cifar10_krizh26.model")])
    assert sgd.cfg.minibatch_size == 8 and sgd.cfg.l2_reg_coef == 0.0


def test_synthetic_split_of_a_data_file_takes_the_shape_of_the_model():
    sgd = train_cifar10.main(TINY + ["--data", os.path.join(ROOT, "examples", "synthetic_cifar10.data"),
                                     "--valid-iters", "1"])
    assert sgd.engine.iter == 3 and len(sgd.valid_history) == 1


def test_ragged_images_train_through_the_common_driver():
    """Samples of different sizes reach the variable-size input operator as (padded rows, size table) batches."""
    import numpy as np
    from rembrandt_b200.cli.common import base_parser, run_training
    from rembrandt_b200.data import RaggedBatchIter
    from rembrandt_b200.models import zoo

    class Ragged:
        dims = (48, 48, 3)

        def __len__(self):
            return 24

        def __getitem__(self, i):
            rng = np.random.default_rng(i)
            h, w = 36 + (i * 5) % 12, 36 + (i * 7) % 12
            return rng.integers(0, 256, (3, h, w), dtype=np.uint8), i % 10

    batches = list(RaggedBatchIter([Ragged()[i] for i in range(6)], 3, (48, 48, 3)))
    (padded, shapes), labels = batches[1]
    assert padded.shape == (3, 3 * 48 * 48) and shapes.tolist() == [[Ragged()[i][0].shape[2], Ragged()[i][0].shape[1]]
                                                                   for i in (3, 4, 5)]
    assert labels.tolist() == [3, 4, 5]
    img = Ragged()[4][0]
    assert np.array_equal(padded[1, : img.size].numpy(), img.reshape(-1))
    args = base_parser("ragged").parse_args(["--device", "cpu", "--batch", "3", "--iters", "2", "--display-iters", "1",
                                             "--valid-iters", "1"])
    cfg = zoo.resnet18_var(num_classes=10, in_hw=32, scale=(36, 40), max_hw=48)
    sgd = run_training(args, cfg, source=Ragged(), valid_source=Ragged())
    assert sgd.engine.iter == 2 and len(sgd.valid_history) == 1


def test_imagenet_tool_on_a_jpeg_record_store_of_ragged_images(tmp_path, monkeypatch):
    """The data path of the reference's enabled ImageNet binary: a record store of JPEG images of different sizes with
    little-endian labels, the variable-size ResNet-18, gradients synchronised then stepped."""
    PIL = pytest.importorskip("PIL.Image")
    import io
    import struct
    import numpy as np
    from rembrandt_b200.cli import dist_train_imagenet
    from rembrandt_b200.data.recorddb import RecordDbWriter
    from rembrandt_b200.models import zoo
    rng = np.random.default_rng(1)
    with RecordDbWriter(str(tmp_path / "imgs")) as wd, RecordDbWriter(str(tmp_path / "lbls")) as wl:
        for i in range(12):
            h, w = 36 + (i * 5) % 12, 36 + (i * 7) % 12
            buf = io.BytesIO()
            PIL.fromarray(rng.integers(0, 256, (h, w, 3), dtype=np.uint8), "RGB").save(buf, format="JPEG")
            wd.append(buf.getvalue())
            wl.append(struct.pack("<i", i % 10))
    (tmp_path / "in.data").write_text(f'[dataset.train]\nsource = "varraydb"\ndata_path = "{tmp_path / "imgs"}"\n'
                                      f'labels_path = "{tmp_path / "lbls"}"\n')
    full = zoo.resnet18_var
    monkeypatch.setattr(zoo, "resnet18_var", lambda: full(num_classes=10, in_hw=32, scale=(36, 40), max_hw=48))
    sgd = dist_train_imagenet.main(["--device", "cpu", "--batch", "2", "--minibatch", "4", "--iters", "2",
                                    "--display-iters", "1", "--model", "resnet18_var", "--data", str(tmp_path / "in.data")])
    assert sgd.engine.iter == 2 and sgd.engine.accum == 2
    # the same run with the JPEG decode spread over three threads draws the same samples in the same order
    again = dist_train_imagenet.main(["--device", "cpu", "--batch", "2", "--minibatch", "4", "--iters", "2",
                                      "--display-iters", "1", "--model", "resnet18_var", "--data", str(tmp_path / "in.data"),
                                      "--decode-threads", "3"])
    assert [h[1] for h in again.history] == pytest.approx([h[1] for h in sgd.history], rel=1e-5)


def test_loader_benchmark_runs_and_the_native_loader_wins():
    from rembrandt_b200.cli import bench_loader
    rows = bench_loader.main(["--shape", "3", "32", "32", "--samples", "512", "--batch", "32", "--batches", "16",
                              "--threads", "2"])
    by = {r["loader"]: r["images_per_s"] for r in rows}
    assert by["native x2"] > by["python iterators"] > 0
    rows = bench_loader.main(["--lmdb", "--shape", "3", "16", "16", "--samples", "256", "--batch", "32", "--batches", "8",
                              "--threads", "2"])
    assert {r["loader"] for r in rows} == {"native lmdb x2", "python lmdb cursor"}


def test_array_backed_sources_use_the_native_loader_by_default(tmp_path, monkeypatch):
    import numpy as np
    from rembrandt_b200.data import native_loader
    rng = np.random.default_rng(3)
    recs = rng.integers(0, 256, (64, 3073), dtype=np.uint8)
    recs[:, 0] %= 10
    (tmp_path / "batch.bin").write_bytes(recs.tobytes())
    (tmp_path / "c.data").write_text(f'[dataset.train]\nsource = "cifar10"\ndata_path = "{tmp_path / "batch.bin"}"\n')
    made = []
    real = native_loader.NativeBatchLoader.__init__

    def spy(self, *a, **k):
        made.append(k.get("threads"))
        return real(self, *a, **k)
    monkeypatch.setattr(native_loader.NativeBatchLoader, "__init__", spy)
    assert train_cifar10.main(TINY + ["--data", str(tmp_path / "c.data")]).engine.iter == 3
    assert made == [2]
    assert train_cifar10.main(TINY + ["--data", str(tmp_path / "c.data"), "--native-loader", "0"]).engine.iter == 3
    assert made == [2]
