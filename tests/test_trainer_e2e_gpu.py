"""End-to-end trainer runs through the launcher, one per architecture / feature path, on 2 GPUs:

    bash runner/primus-cli direct --gpus 2 --log_file <log> -- train pretrain --config tests/trainer_e2e.yaml

Three iterations of a small model on mock data; a run passes when the log carries the completion line and three
finite losses (the scheme of the reference's trainer tests, tests/trainer/test_megatron_trainer.py:55-87,133-149)."""
import math
import os
import re
import subprocess

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CLI = os.path.join(ROOT, "runner", "primus-cli")
CFG = os.path.join(ROOT, "tests", "trainer_e2e.yaml")

CASES = {
    "llama_dp2_mxfp8": dict(gpus=2, env=dict(PRIMUS_FP8="e4m3")),
    "llama_tp2_sp": dict(gpus=2, env=dict(PRIMUS_TP="2", PRIMUS_SP="true")),
    "llama_tp2_sp_mxfp8_overlap": dict(gpus=2, env=dict(PRIMUS_TP="2", PRIMUS_SP="true", PRIMUS_FP8="e4m3",
                                                        PRIMUS_TP_OVERLAP="true")),
    "llama_pp2_1f1b": dict(gpus=2, env=dict(PRIMUS_PP="2")),
    "llama_pp2_interleaved": dict(gpus=2, env=dict(PRIMUS_PP="2", PRIMUS_VPP="2", PRIMUS_PP_ALGO="interleaved")),
    "llama_pp2_zerobubble": dict(gpus=2, env=dict(PRIMUS_PP="2", PRIMUS_PP_ALGO="zerobubble")),
    "llama_cp2_a2a": dict(gpus=2, env=dict(PRIMUS_CP="2")),
    "llama_cp2_ring": dict(gpus=2, env=dict(PRIMUS_CP="2", PRIMUS_CP_COMM="p2p")),
    "llama_recompute_uniform": dict(gpus=1, env=dict(PRIMUS_RECOMPUTE="full", PRIMUS_RECOMPUTE_METHOD="uniform",
                                                     PRIMUS_RECOMPUTE_LAYERS="2")),
    "llama_dp2_fused_dp": dict(gpus=2, env=dict(PRIMUS_FUSED_DP="true")),
    "moe_ep2": dict(gpus=2, env=dict(PRIMUS_MODEL="moe_proxy_single_node.yaml", PRIMUS_EP="2", PRIMUS_NUM_LAYERS="2", PRIMUS_MOE_LAYER_FREQ="[0, 1]")),
    "moe_ep2_mxfp8": dict(gpus=2, env=dict(PRIMUS_MODEL="moe_proxy_single_node.yaml", PRIMUS_EP="2", PRIMUS_NUM_LAYERS="2", PRIMUS_MOE_LAYER_FREQ="[0, 1]",
                                           PRIMUS_FP8="e4m3")),
    "moe_ep2_fused": dict(gpus=2, env=dict(PRIMUS_MODEL="moe_proxy_single_node.yaml", PRIMUS_EP="2", PRIMUS_NUM_LAYERS="2", PRIMUS_MOE_LAYER_FREQ="[0, 1]",
                                           PRIMUS_MEGA_MOE="true")),
    "deepseek_v2_lite_mla_ep2": dict(gpus=2, env=dict(PRIMUS_MODEL="deepseek_v2_lite.yaml", PRIMUS_EP="2",
                                                      PRIMUS_NUM_LAYERS="2", PRIMUS_MOE_LAYER_FREQ="[0, 1]")),
    "qwen3_30B_A3B_ep2": dict(gpus=2, env=dict(PRIMUS_MODEL="qwen3_30B_A3B.yaml", PRIMUS_EP="2", PRIMUS_NUM_LAYERS="2")),
    "gpt_oss_sink_attention": dict(gpus=1, env=dict(PRIMUS_MODEL="gpt_oss_20B.yaml", PRIMUS_NUM_LAYERS="2")),
}


@pytest.mark.parametrize("name", sorted(CASES))
def test_trainer_through_launcher(name, tmp_path):
    case = CASES[name]
    if torch.cuda.device_count() < case["gpus"]:
        pytest.skip(f"needs {case['gpus']} GPUs")
    log = tmp_path / "train.log"
    env = dict(os.environ)
    env.pop("SLURM_JOB_ID", None)
    env.update(PRIMUS_WORKSPACE=str(tmp_path / "out"), PRIMUS_EXP_NAME=name, MASTER_ADDR="127.0.0.1",
               NCCL_NVLS_ENABLE="0", PYTHONPATH=ROOT + os.pathsep + env.get("PYTHONPATH", ""))
    env.update(case["env"])
    cmd = ["bash", CLI, "direct", "--gpus", str(case["gpus"]), "--no-numa", "--master_addr", "127.0.0.1",
           "--log_file", str(log), "--", "train", "pretrain", "--config", CFG]
    r = subprocess.run(cmd, capture_output=True, text=True, env=env, cwd=ROOT, timeout=600)
    text = log.read_text() if log.exists() else ""
    tail = (text or r.stdout + r.stderr)[-3000:]
    assert r.returncode == 0, f"{name}: exit {r.returncode}\n{tail}"
    assert "Training completed." in text, f"{name}: no completion line\n{tail}"
    losses = [float(x) for x in re.findall(r"lm loss: ([0-9.eE+-]+)", text)]
    assert len(losses) >= 3 and all(math.isfinite(l) and 0 < l < 20 for l in losses), (name, losses)
