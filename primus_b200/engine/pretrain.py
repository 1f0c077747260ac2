"""``PretrainTrainer``: the trainer the CLI runs for ``train pretrain``.  It maps the resolved
experiment parameters onto :class:`TransformerConfig` / :class:`TrainConfig`, initialises the process
groups and drives :class:`primus_b200.engine.trainer.Trainer`
(counterpart of primus/backends/megatron/megatron_pretrain_trainer.py:128-291 in the reference)."""
from __future__ import annotations

import os

import torch

from ..core.utils import logger as logutil
from ..models.config import TransformerConfig
from ..parallel import state as ps
from .base_trainer import BaseTrainer
from .trainer import init_parallel_state, TrainConfig, Trainer

COMPLETED_MESSAGE = "Training completed."


class PretrainTrainer(BaseTrainer):
    def setup(self):
        p = self.params
        backend = p.get("distributed_backend", "nccl")
        if not torch.cuda.is_available():
            backend = "gloo"
        if self.world_size > 1 or "RANK" in os.environ:
            ps.init_distributed(backend, float(p.get("distributed_timeout_minutes", 10)))
        if torch.cuda.is_available():
            torch.cuda.set_device(self.local_rank)

    def build_configs(self):
        p = self.params
        mcfg = TransformerConfig.from_dict(p)
        tcfg = TrainConfig.from_dict(p)
        return mcfg, tcfg

    def init(self):
        mcfg, tcfg = self.build_configs()
        init_parallel_state(mcfg, tcfg)
        self.engine = Trainer(mcfg, tcfg, log_fn=logutil.log_rank_all)
        if tcfg.load:
            self.engine.load_checkpoint()
        if tcfg.pretrained_hf_path and self.engine.iteration == 0:
            # start from published Hugging Face weights (every rank reads the files and keeps its own slices)
            from . import hf_convert

            hf_convert.load_hf_into_trainer(self.engine, tcfg.pretrained_hf_path)
            logutil.log_rank_0(f"loaded Hugging Face weights from {tcfg.pretrained_hf_path}")
        logutil.log_rank_0(f"model parameters: {mcfg.num_parameters() / 1e9:.3f} B; "
                           f"dp={ps.dp_size()} tp={ps.tp_size()} pp={ps.pp_size()} ep={ps.ep_size()}")

    def convert_checkpoint(self) -> str:
        """``ckpt_convert_format`` / ``ckpt_convert_save``: the loaded state written in the other checkpoint format."""
        tc = self.engine.tcfg
        if not tc.load or not tc.ckpt_convert_save:
            raise ValueError("ckpt_convert_format needs load (the checkpoint to read) and ckpt_convert_save (where to write)")
        was = tc.ckpt_format
        tc.ckpt_format = tc.ckpt_convert_format
        try:
            d = self.engine.save_checkpoint(tc.ckpt_convert_save)
        finally:
            tc.ckpt_format = was
        logutil.log_rank_0(f"converted the checkpoint of iteration {self.engine.iteration} from {tc.load} to "
                           f"{tc.ckpt_convert_format} format in {d}")
        return d

    def train(self):
        if self.engine.tcfg.ckpt_convert_format:
            self.convert_checkpoint()
            logutil.log_rank_0(COMPLETED_MESSAGE)
            return

        def publish(tr, loss):
            if self.runtime_state is not None:
                self.runtime_state.update_metrics(**tr.last_metrics)

        self.losses = self.engine.train(on_step=publish)
        tc = self.engine.tcfg
        if tc.save and not self.params.get("disable_last_saving", False):
            self.engine.save_checkpoint()
        if tc.export_hf_path:
            from . import hf_convert

            hf_convert.export_trainer_to_hf(self.engine, tc.export_hf_path)
        logutil.log_rank_0(COMPLETED_MESSAGE)

    def cleanup(self):
        import torch.distributed as dist

        if dist.is_initialized():
            dist.barrier()
            if os.environ.get("PRIMUS_EXIT_FAST") == "1":
                os._exit(0)
            dist.destroy_process_group()
            ps.destroy_model_parallel()
