"""EM optimizers over a :class:`TensorCircuit` (PyJuice: optim/optim.py:7-142, optim/mini_batch_em.py:9-56).

The "gradient" of a circuit is its parameter flows, accumulated by ``pc.backward``; ``step`` turns them into
an EM update and clears the accumulators.  With ``ddp=True`` the flows of all ranks are summed first, so every
rank applies the identical update.
"""
from __future__ import annotations

from typing import Optional

import torch

from .model import TensorCircuit


class CircuitOptimizer:
    def __init__(self, pc: TensorCircuit, pseudocount: float = 0.0, keep_zero_params: bool = False,
                 ddp: bool = False, ddp_dtype: Optional[torch.dtype] = None, ddp_group=None, sync_every: int = 1):
        assert sync_every >= 1, "`sync_every` should be a positive integer."
        if sync_every != 1:
            raise NotImplementedError("only synchronous data parallelism (`sync_every=1`) is on the compiled path")
        self.pc = pc
        self.pseudocount = pseudocount
        self.keep_zero_params = keep_zero_params
        self.ddp, self.ddp_dtype, self.ddp_group = ddp, ddp_dtype, ddp_group
        self.sync_every = sync_every
        self._update_count = 0
        self.pc._optim_hyperparams["flows_memory"] = 1.0     # backward passes accumulate within an update window
        self.zero_flows()

    def zero_flows(self):
        self.pc.init_param_flows(flows_memory=0.0)

    def _sync_flows(self):
        if self.ddp:
            self.pc.sync_param_flows(dtype=self.ddp_dtype, group=self.ddp_group)

    def step(self, step_size: Optional[float] = None):
        raise NotImplementedError("`step` must be implemented by a CircuitOptimizer subclass.")


class MiniBatchEM(CircuitOptimizer):
    """EM update every ``niters_per_update`` mini-batches:
    ``params <- (1 - step_size) * params + step_size * new_params``."""

    def __init__(self, pc: TensorCircuit, step_size: float = 0.1, niters_per_update: int = 1, pseudocount: float = 0.0,
                 keep_zero_params: bool = False, ddp: bool = False, ddp_dtype: Optional[torch.dtype] = None,
                 ddp_group=None, sync_every: int = 1):
        assert 0.0 < step_size <= 1.0, "`step_size` should be in (0, 1]."
        assert niters_per_update >= 1, "`niters_per_update` should be a positive integer."
        super().__init__(pc, pseudocount=pseudocount, keep_zero_params=keep_zero_params, ddp=ddp,
                         ddp_dtype=ddp_dtype, ddp_group=ddp_group, sync_every=sync_every)
        self.step_size = step_size
        self.niters_per_update = niters_per_update
        self._iter = 0
        if ddp and niters_per_update == 1 and ddp_dtype in (None, torch.float32):
            pc.enable_flow_sync_overlap(ddp_group)       # every backward pass is followed by a sync: overlap it

    def step(self, step_size: Optional[float] = None):
        self._iter += 1
        if self._iter % self.niters_per_update != 0:
            return
        self._sync_flows()
        ss = self.step_size if step_size is None else step_size
        self.pc.mini_batch_em(step_size=ss, pseudocount=self.pseudocount, keep_zero_params=self.keep_zero_params)
        self.zero_flows()
        self._update_count += 1


class FullBatchEM(MiniBatchEM):
    """Full-batch EM: accumulate over the whole pass, then ``step()`` replaces the parameters (step size 1)."""

    def __init__(self, pc: TensorCircuit, pseudocount: float = 0.0, keep_zero_params: bool = False, **kwargs):
        super().__init__(pc, step_size=1.0, niters_per_update=1, pseudocount=pseudocount,
                         keep_zero_params=keep_zero_params, **kwargs)
        pc._overlap_group = None      # many backward passes per step: the flows must not be reduced after the first
