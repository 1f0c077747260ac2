"""Launcher (bash) through --dry-run: mode dispatch, config precedence, hooks protocol, validation; Python CLI."""
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CLI = os.path.join(ROOT, "primus-cli")


def run(args, env=None, cwd=ROOT):
    e = dict(os.environ)
    e.pop("SLURM_JOB_ID", None)
    e.update(env or {})
    return subprocess.run(["bash", CLI, *args], capture_output=True, text=True, env=e, cwd=cwd)


def test_direct_dry_run_builds_torchrun():
    r = run(["--dry-run", "direct", "--gpus", "4", "--nnodes", "2", "--node_rank", "1", "--master_addr", "10.0.0.1",
             "--master_port", "2345", "--no-numa", "--", "train", "pretrain", "--config", "x.yaml", "--lr", "0.1"])
    assert r.returncode == 0, r.stderr
    line = [l for l in r.stdout.splitlines() if l.startswith("[dry-run] torchrun")][0]
    for tok in ("--nproc_per_node 4", "--nnodes 2", "--node_rank 1", "--master_addr 10.0.0.1", "--master_port 2345",
                "train pretrain --config x.yaml --lr 0.1"):
        assert tok in line, line


def test_exit_codes_and_usage_errors():
    assert run([]).returncode == 2
    assert run(["bogus-mode"]).returncode == 2
    assert run(["--dry-run", "direct"]).returncode == 2                      # no primus args
    assert run(["--dry-run", "direct", "--gpus", "99", "--", "train"]).returncode == 2
    assert run(["--dry-run", "direct", "--env", "NOEQUALS", "--", "train"]).returncode == 2
    assert run(["--help"]).returncode == 0


def test_config_precedence_cli_over_user_over_system(tmp_path):
    user = tmp_path / "user.yaml"
    user.write_text("direct:\n  gpus_per_node: 2\n  master_port: 4444\n")
    r = run(["--dry-run", "--config", str(user), "direct", "--no-numa", "--", "train", "pretrain", "--config", "x"],
            env={"GPUS_PER_NODE": "", "MASTER_PORT": ""})
    assert "--nproc_per_node 2" in r.stdout and "--master_port 4444" in r.stdout, r.stdout + r.stderr
    r = run(["--dry-run", "--config", str(user), "direct", "--gpus", "3", "--no-numa", "--", "train", "pretrain",
             "--config", "x"], env={"GPUS_PER_NODE": "", "MASTER_PORT": ""})
    assert "--nproc_per_node 3" in r.stdout


def test_hooks_env_and_extra_protocol(tmp_path):
    hooks = tmp_path / "hooks"
    (hooks / "train" / "pretrain").mkdir(parents=True)
    (hooks / "00_global.sh").write_text("echo env.PB_HOOK_VAR=42\necho extra.seed=7\necho plain message\n")
    (hooks / "train" / "pretrain" / "10_specific.sh").write_text("echo extra.train_iters=3\n")
    r = run(["--dry-run", "direct", "--single", "--", "train", "pretrain", "--config", "x"],
            env={"PRIMUS_HOOKS_DIR": str(hooks)})
    assert r.returncode == 0, r.stderr
    assert "--seed 7" in r.stdout and "--train_iters 3" in r.stdout
    assert "plain message" in r.stderr
    (hooks / "99_fail.sh").write_text("exit 3\n")
    assert run(["--dry-run", "direct", "--single", "--", "train", "pretrain", "--config", "x"],
               env={"PRIMUS_HOOKS_DIR": str(hooks)}).returncode == 1


def test_container_and_slurm_command_synthesis():
    r = run(["--dry-run", "container", "--image", "img:1", "--volume", "/data:/data", "--shm-size", "32g", "--privileged",
             "--", "train", "pretrain", "--config", "x"])
    assert r.returncode == 0, r.stderr
    assert "docker run --rm" in r.stdout and "--shm-size 32g" in r.stdout and "--volume /data:/data" in r.stdout
    assert "--privileged" in r.stdout and "img:1 bash" in r.stdout and "direct -- train pretrain" in r.stdout
    assert run(["--dry-run", "container", "--memory", "lots", "--image", "i", "--", "train"]).returncode == 2
    r = run(["--dry-run", "slurm", "sbatch", "-N", "2", "--time", "1:00:00", "--", "train", "pretrain", "--config", "x"])
    assert r.returncode == 0 and "sbatch -N 2 --time 1:00:00" in r.stdout and "primus-cli-slurm-entry.sh" in r.stdout
    r = run(["--dry-run", "slurm", "--", "direct", "--gpus", "8", "--", "benchmark", "gemm"])
    assert "srun" in r.stdout and "--nodes 1" in r.stdout


def test_python_cli_help_and_dry_run(tmp_path):
    env = dict(os.environ, PYTHONPATH=ROOT, PRIMUS_WORKSPACE=str(tmp_path))
    r = subprocess.run([sys.executable, "-m", "primus_b200.cli.main", "--help"], capture_output=True, text=True, env=env)
    assert r.returncode == 0 and "train" in r.stdout and "projection" in r.stdout
    cfg = os.path.join(ROOT, "examples", "configs", "llama_tiny-pretrain.yaml")
    r = subprocess.run([sys.executable, "-m", "primus_b200.cli.main", "train", "pretrain", "--config", cfg, "--dry-run",
                        "--train_iters", "5"], capture_output=True, text=True, env=env)
    assert r.returncode == 0, r.stderr
    assert "train_iters: 5" in r.stdout
    r = subprocess.run([sys.executable, "-m", "primus_b200.cli.main", "benchmark", "--nope"], capture_output=True,
                       text=True, env=env)
    assert r.returncode != 0


def test_direct_mode_really_trains_on_cpu(tmp_path):
    """Not a dry run: the launcher starts the worker script, which trains a tiny model for two iterations on the CPU
    and leaves the completion line in the log file."""
    log = tmp_path / "train.log"
    r = run(["direct", "--single", "--log_file", str(log), "--", "train", "pretrain", "--config",
             os.path.join(ROOT, "tests", "trainer_e2e.yaml")],
            env={"CUDA_VISIBLE_DEVICES": "", "PRIMUS_WORKSPACE": str(tmp_path / "out"), "PRIMUS_NUM_LAYERS": "2",
                 "PRIMUS_SEQ": "64", "PRIMUS_GBS": "2", "PRIMUS_TRAIN_ITERS": "2", "PRIMUS_OVERLAP": "false"})
    text = log.read_text() if log.exists() else ""
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "Training completed." in text and text.count("lm loss:") == 2, text[-2000:]


def test_deps_check_reports_toolchain_packages_and_native_library():
    import subprocess

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run(["bash", os.path.join(root, "runner", "primus-cli"), "deps", "check"], capture_output=True, text=True,
                       timeout=300)
    assert "torch" in r.stdout and "native library" in r.stdout and "python3" in r.stdout, r.stdout + r.stderr
    assert r.returncode in (0, 1)           # 1: something is missing or stale on this machine; the report still prints
