"""Layer runner: gradient checkpointing, FSDP gather/reduce-scatter and activation offload in one autograd node.

On multi-rank CUDA runs the next layer's all-gather is started on a side stream when a layer begins (forward: layer i + 1,
backward: layer i - 1) and a layer's gradient reduce-scatter runs on that stream under the backward of the layer before it.

Forward of a layer: all-gather its parameter unit, run it without building a graph, stash its input (optionally to
pinned host memory on a side stream), free the gathered parameters. Backward: gather again, bring the input back
(prefetching the next layer's input while this one recomputes), recompute with a graph, backpropagate, reduce-scatter
the unit's gradients, free. (Upstream: verl FSDP2 + checkpoint wrappers, ``3rdparty/verl/patches/0032-*`` for the
offload of checkpoint inputs and ``0026-*`` for retaining attention outputs inside a checkpoint.)
"""

from __future__ import annotations

from typing import Optional

import torch


class LayerRunner:
    """Callable ``(index, layer, residual, meta) -> residual`` installed on the model as ``layer_runner``."""

    def __init__(self, sharded=None, offload=None, checkpoint: bool = True, retain_attention: bool = False, skip_down_proj: bool = False):
        self.sharded = sharded
        self.offload = offload
        self.checkpoint = checkpoint
        # keep the attention outputs of the graph-free pass for the recompute pass (GPU attention kernel only)
        self.retain_attention = retain_attention
        # the recompute pass skips the forward of the layer's last GEMM (its value is never read there)
        self.skip_down_proj = skip_down_proj
        self.last_micro_batch = True

    def unit(self, i: int):
        return self.sharded.layer_units[i] if self.sharded is not None else None

    def prefetch(self, i: int) -> None:
        """Start the all-gather of layer ``i``'s parameters while the current layer computes."""
        if self.sharded is not None and 0 <= i < len(self.sharded.layer_units):
            self.sharded.layer_units[i].prefetch()

    def __call__(self, i: int, layer, r: torch.Tensor, meta) -> torch.Tensor:
        if not torch.is_grad_enabled() or not self.checkpoint:
            u = self.unit(i)
            if u is not None:
                u.gather()
                self.prefetch(i + 1)
            out = layer(r, meta)
            if u is not None and not torch.is_grad_enabled():
                u.release()
            return out
        if not r.requires_grad:
            r = r.detach().requires_grad_(True)  # the node must be part of the graph even when the embedding is frozen
        return _CheckpointedLayer.apply(r, self, i, layer, meta)


class _CheckpointedLayer(torch.autograd.Function):
    @staticmethod
    def forward(ctx, r, runner: LayerRunner, i: int, layer, meta):
        u = runner.unit(i)
        if u is not None:
            u.gather()
            runner.prefetch(i + 1)
        ctx.attn_box = [] if runner.retain_attention else None
        with torch.no_grad():
            if ctx.attn_box is not None:
                from ..ops.attention import retain_attention

                with retain_attention("record", ctx.attn_box):
                    out = layer(r, meta)
            else:
                out = layer(r, meta)
        if u is not None:
            u.release()
        ctx.runner, ctx.i, ctx.layer, ctx.meta = runner, i, layer, meta
        if runner.offload is not None:
            ctx.handle = runner.offload.stash(i, r)
            ctx.saved = None
        else:
            ctx.handle = None
            ctx.saved = r.detach()
        return out

    @staticmethod
    def backward(ctx, grad_out):
        runner, i, layer, meta = ctx.runner, ctx.i, ctx.layer, ctx.meta
        u = runner.unit(i)
        if u is not None:
            u.gather()
            runner.prefetch(i - 1)
        if ctx.handle is not None:
            r = runner.offload.fetch(ctx.handle)
            runner.offload.prefetch(i - 1)
        else:
            r = ctx.saved
        r = r.detach().requires_grad_(True)
        from ..models import hybrid

        prev_skip, hybrid.RECOMPUTE["skip_down_proj"] = hybrid.RECOMPUTE["skip_down_proj"], runner.skip_down_proj
        with torch.enable_grad():
            if ctx.attn_box:
                from ..ops.attention import retain_attention

                with retain_attention("replay", ctx.attn_box):
                    out = layer(r, meta)
            else:
                out = layer(r, meta)
        hybrid.RECOMPUTE["skip_down_proj"] = prev_skip
        torch.autograd.backward(out, grad_out)
        if u is not None:
            u.reduce_grads(runner.last_micro_batch)
            u.release()
        return r.grad, None, None, None, None


def install(model, runner: Optional[LayerRunner]) -> None:
    model.layer_runner = runner
