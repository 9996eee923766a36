"""Shared helpers of the GPU parity tests: run the CUDA path and the CPU oracle on the same circuit and inputs."""
import torch

from oracle import pc_oracle as orc

LL_ATOL = 1e-3          # nats, absolute, per-sample log-likelihood
REL_TOL = 1e-3          # relative, node flows / parameter flows / post-EM parameters


def rel_close(got: torch.Tensor, ref: torch.Tensor, rtol: float = REL_TOL, floor: float = 1e-6):
    """|got - ref| <= rtol * max(|ref|, floor * scale) elementwise, scale = largest reference magnitude."""
    got, ref = got.double().cpu(), ref.double().cpu()
    scale = max(ref.abs().max().item(), 1e-30)
    err = (got - ref).abs()
    bound = rtol * torch.clamp(ref.abs(), min=floor * scale)
    bad = err > bound
    return not bool(bad.any()), (err / torch.clamp(ref.abs(), min=floor * scale)).max().item()


def oracle_step(pc, x, step=None, pseudo=0.0, params=None, input_params=None, ll_weights=None):
    params = pc.params.data if params is None else params
    iparams = [l.params.data for l in pc.input_layer_group] if input_params is None else input_params
    lls, st = orc.forward(pc, x.cpu(), params, iparams)
    orc.backward(pc, x.cpu(), params, iparams, st, ll_weights=ll_weights)
    new = orc.em_update(pc, params, iparams, st, step, pseudo) if step is not None else None
    return lls, st, new


def folded_input_flows(layer, flows):
    """Input-layer flows with every tied group's accumulators summed into its source range (replicas zero)."""
    f = flows.detach().double().cpu().clone()
    for start, n, ch in layer.tied2source_nids:
        start, n = int(start), int(n)
        tot = sum(f[int(c):int(c) + n].clone() for c in ch)
        for c in ch:
            f[int(c):int(c) + n] = 0.0
        f[start:start + n] = tot
    return f


def check_against_oracle(pc, x, step=0.1, pseudo=0.1, logspace_flows=True, rtol=REL_TOL, fold_input_flows=False):
    """One forward + backward + EM step on the GPU, compared with the oracle.  Returns a dict of worst errors.
    ``fold_input_flows``: compare the input layers' flows after summing the accumulators of every tied group (layers
    that accumulate through a transposed shadow table report the flows of tied replicas in the source range)."""
    dev = pc.device
    p0 = pc.params.data.detach().cpu().clone()
    ip0 = [l.params.data.detach().cpu().clone() for l in pc.input_layer_group]
    ref_lls, st, (ref_p, ref_ip) = oracle_step(pc, x, step, pseudo, params=p0, input_params=ip0)

    pc.init_param_flows(flows_memory=0.0)
    lls = pc(x.to(dev))
    pc.backward(x.to(dev), logspace_flows=logspace_flows)
    out = {}
    out["ll"] = (lls.double().cpu() - ref_lls).abs().max().item()
    assert out["ll"] <= LL_ATOL, f"log-likelihood off by {out['ll']} nats"

    nf = pc.node_flows.double().cpu()
    nf = nf.exp() if logspace_flows else nf
    ok, out["node_flows"] = rel_close(nf[pc.num_dummy_nodes:], st.node_flows.exp()[pc.num_dummy_nodes:], rtol)
    assert ok, f"node flows rel err {out['node_flows']}"
    ok, out["param_flows"] = rel_close(pc.param_flows, st.param_flows, rtol)
    assert ok, f"sum parameter flows rel err {out['param_flows']}"
    for layer, ref in zip(pc.input_layer_group, st.input_param_flows):
        got = layer.param_flows
        if fold_input_flows:
            got, ref = folded_input_flows(layer, got), folded_input_flows(layer, ref)
        ok, out["input_flows"] = rel_close(got, ref, rtol)
        assert ok, f"input parameter flows rel err {out['input_flows']}"

    pc.mini_batch_em(step_size=step, pseudocount=pseudo)
    ok, out["params"] = rel_close(pc.params.data[pc.num_dummy_params:], ref_p[pc.num_dummy_params:], rtol)
    assert ok, f"post-EM sum parameters rel err {out['params']}"
    for layer, ref in zip(pc.input_layer_group, ref_ip):
        ok, out["input_params"] = rel_close(layer.params.data, ref, rtol)
        assert ok, f"post-EM input parameters rel err {out['input_params']}"
    torch.cuda.synchronize()
    return out


def fold_tied_flows_(pc, param_flows, input_param_flows):
    """In place on oracle-side accumulators: every tied group's source range += its replica accumulators, replicas = 0
    (what `pcx_tied_accum` does on the device before an EM update)."""
    for start, n, accs in pc._tied_sum_groups:
        tot = sum(param_flows[a:a + n].clone() for a in accs)
        for a in accs:
            param_flows[a:a + n] = 0.0
        param_flows[start:start + n] = tot
    for layer, pf in zip(pc.input_layer_group, input_param_flows):
        for start, n, ch in layer.tied2source_nids:
            start, n = int(start), int(n)
            tot = sum(pf[int(c):int(c) + n].clone() for c in ch)
            for c in ch:
                pf[int(c):int(c) + n] = 0.0
            pf[start:start + n] = tot


class OracleTrainer:
    """CPU-side mirror of a training loop: parameters and accumulated flows carried from step to step."""

    def __init__(self, pc):
        self.pc = pc
        self.params = pc.params.data.detach().cpu().double().clone()
        self.iparams = [l.params.data.detach().cpu().double().clone() for l in pc.input_layer_group]
        self.pf = torch.zeros(pc.num_param_flows, dtype=torch.float64)
        self.ipf = [torch.zeros(l.num_param_flows, dtype=torch.float64) for l in pc.input_layer_group]

    def accumulate(self, x, flows_memory=1.0):
        """One forward + backward pass: flows *= flows_memory, then += the flows of ``x``.  Returns the LLs."""
        self.pf *= flows_memory
        for f in self.ipf:
            f *= flows_memory
        lls, st = orc.forward(self.pc, x.cpu(), self.params, self.iparams)
        orc.backward(self.pc, x.cpu(), self.params, self.iparams, st, param_flows=self.pf, input_param_flows=self.ipf)
        self.pf, self.ipf = st.param_flows, st.input_param_flows
        self._st = st
        return lls

    def update(self, step_size, pseudocount, zero_flows=True):
        fold_tied_flows_(self.pc, self.pf, self.ipf)
        self._st.param_flows, self._st.input_param_flows = self.pf, self.ipf
        self.params, self.iparams = orc.em_update(self.pc, self.params, self.iparams, self._st, step_size, pseudocount)
        if zero_flows:
            self.pf.zero_()
            for f in self.ipf:
                f.zero_()

    def check_params(self, pc, rtol=REL_TOL):
        ok, err = rel_close(pc.params.data[pc.num_dummy_params:], self.params[pc.num_dummy_params:], rtol)
        assert ok, f"sum parameters rel err {err}"
        worst = err
        for layer, ref in zip(pc.input_layer_group, self.iparams):
            ok, err = rel_close(layer.params.data, ref, rtol)
            assert ok, f"input parameters rel err {err}"
            worst = max(worst, err)
        return worst
