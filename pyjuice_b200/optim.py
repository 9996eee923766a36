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
            self.pc.sync_param_flows(dtype=self.ddp_dtype, group=self.ddp_group, _lazy=True)

    def _average_params(self):
        """Local-SGD: every rank's parameters become their mean over the process group (a mean of normalised
        parameter vectors is normalised, so nothing is renormalised).  PyJuice: optim/optim.py:99-124."""
        if self.ddp:
            self.pc.average_params(dtype=self.ddp_dtype, group=self.ddp_group)

    def _post_update_sync(self):
        """Called after each local EM update: with ``sync_every > 1`` the ranks update on their own flows and
        average their parameters every ``sync_every`` updates (PyJuice: optim/optim.py:126-132)."""
        self._update_count += 1
        if self.sync_every > 1 and self._update_count % self.sync_every == 0:
            self._average_params()

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
        if ddp and sync_every == 1 and niters_per_update == 1:
            pc.enable_flow_sync_overlap(ddp_group, ddp_dtype)     # every backward pass is followed by a sync: overlap it
        else:
            pc._overlap_group = None

    def step(self, step_size: Optional[float] = None):
        self._iter += 1
        if self._iter % self.niters_per_update != 0:
            return
        if self.sync_every <= 1:
            self._sync_flows()           # synchronous data parallelism: one update on the summed flows
        ss = self.step_size if step_size is None else step_size
        self.pc.mini_batch_em(step_size=ss, pseudocount=self.pseudocount, keep_zero_params=self.keep_zero_params)
        self.zero_flows()
        self._post_update_sync()


class FullBatchEM(CircuitOptimizer):
    """Full-batch EM: flows accumulate over the whole pass, then ``step()`` makes one exact M-step (step size 1
    unless overridden).  PyJuice: optim/full_batch_em.py:21-27."""

    def __init__(self, pc: TensorCircuit, pseudocount: float = 0.0, keep_zero_params: bool = False, **kwargs):
        super().__init__(pc, pseudocount=pseudocount, keep_zero_params=keep_zero_params, **kwargs)
        pc._overlap_group = None      # many backward passes per step: the flows must not be reduced after the first

    def step(self, step_size: Optional[float] = None):
        self._sync_flows()
        ss = 1.0 if step_size is None else step_size
        self.pc.mini_batch_em(step_size=ss, pseudocount=self.pseudocount, keep_zero_params=self.keep_zero_params)
        self.zero_flows()
