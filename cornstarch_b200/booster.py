"""``Booster``: the five-call facade user scripts drive (``boost``, ``execute_pipeline``, ``save_*``, ``load_*``).

Same calls as ``colossalai.booster.Booster`` that the reference examples use
(examples/distributed/run_vlm_hybrid.py:165-209, docs/parallelization/cornstarch_parallel.md:34-52,230-246
in the reference), implemented as a thin layer over the plugin.
"""

from __future__ import annotations

import torch


class Booster:
    def __init__(self, plugin=None, device: str | None = None, mixed_precision=None):
        self.plugin = plugin
        self.checkpoint_io = None

    def boost(self, model, optimizer=None, criterion=None, dataloader=None, lr_scheduler=None, **plugin_kwargs):
        """``plugin_kwargs`` go to the plugin's ``configure`` (``forced=True`` re-plans an already boosted model with the
        heterogeneous plugin)."""
        out = self.plugin.configure(model, optimizer, criterion, dataloader, lr_scheduler, **plugin_kwargs)
        self.checkpoint_io = self.plugin.get_checkpoint_io()
        return out

    def execute_pipeline(self, data_iter, model, criterion, optimizer=None, return_loss: bool = True,
                         return_outputs: bool = False) -> dict:
        return self.plugin.execute_pipeline(data_iter, model, criterion, optimizer, return_loss, return_outputs)

    def backward(self, loss: torch.Tensor, optimizer) -> None:
        optimizer.backward(loss) if hasattr(optimizer, "backward") else loss.backward()

    def no_sync(self, model=None, optimizer=None):
        return model.no_sync()

    # ---- checkpoints
    def save_model(self, model, checkpoint: str, shard: bool = True, gather_dtensor: bool = True, prefix=None,
                   size_per_shard: int = 1024, use_safetensors: bool = True):
        self.checkpoint_io.save_model(model, checkpoint, shard=shard, size_per_shard=size_per_shard, use_safetensors=use_safetensors)

    def load_model(self, model, checkpoint, strict: bool = True):
        return self.checkpoint_io.load_model(model, checkpoint, strict=strict)

    def save_optimizer(self, optimizer, checkpoint: str, shard: bool = True, gather_dtensor: bool = True, prefix=None,
                       size_per_shard: int = 1024):
        self.checkpoint_io.save_optimizer(optimizer, checkpoint, shard=shard, size_per_shard=size_per_shard)

    def load_optimizer(self, optimizer, checkpoint: str):
        return self.checkpoint_io.load_optimizer(optimizer, checkpoint)

    def save_lr_scheduler(self, lr_scheduler, checkpoint: str):
        torch.save(lr_scheduler.state_dict(), checkpoint)

    def load_lr_scheduler(self, lr_scheduler, checkpoint: str):
        lr_scheduler.load_state_dict(torch.load(checkpoint, weights_only=False))
