"""Munazen: a decoder-only model whose layers are either a gated-linear-attention mixer or a softmax-attention mixer and a recurrent
block side by side, with hyper-connections (several residual streams mixed by small learned matrices) in place of the residual sum, an
RMS norm in groups, PolyNorm feed-forwards, and a range of layers that runs several times with the same weights.

The class only DESCRIBES the model with the mechanisms of ``layers``; cache, state slots, batching and the step loop belong to
``seqengine.SequenceEngine``. Tensor names: ``embed``, ``l<i>.norm<q>``, ``l<i>.hc<q>.{in,out,mix}``, ``l<i>.mix.*``, ``l<i>.mlp.*``,
``final.norm``, ``head``."""
from __future__ import annotations

from ..layers import FusedLinear, GatedLinearAttention, GatedLinearRecurrence, GatedRotaryAttention, MixerGroup, PolyNormFeedForward


class _Sublayer:
    def __init__(self, norm_w, hc_in, hc_mix, hc_out, body):
        self.norm_w, self.hc_in, self.hc_mix, self.hc_out, self.body = norm_w, hc_in, hc_mix, hc_out, body


class MunazenModel:
    rotary_layout = 0   # dimension 2i pairs with 2i+1

    def __init__(self, cfg, w, ops, device):
        self.cfg, self.ops, self.device = cfg, ops, device
        self.vocab, self.width, self.streams = cfg.vocab, cfg.width, cfg.streams
        self.embed = w["embed"].contiguous()
        self.final_norm = w["final.norm"].float().contiguous()
        self.head = FusedLinear([(w["head"], None)], ops, device)
        self.runs = cfg.layer_runs()
        self.layers = []
        for i, lc in enumerate(cfg.layers):
            pre = f"l{i}."
            if lc.type == "parallel":
                mixer = MixerGroup([("left", GatedRotaryAttention(lc.left, w, pre + "mix.left.", ops, device, self.rotary_layout), lc.left_scale),
                                    ("right", GatedLinearRecurrence(lc.right, w, pre + "mix.right.", ops, device), lc.right_scale)], ops, device)
            else:
                mixer = MixerGroup([("gla", GatedLinearAttention(lc.gla, w, pre + "mix.", ops, device, cfg.norm_eps), 1.0)], ops, device)
            subs = [self._sublayer(w, pre, 1, mixer)]
            if lc.ff is not None:
                subs.append(self._sublayer(w, pre, 2, PolyNormFeedForward(w, pre + "mlp.", ops, device, cfg.norm_eps)))
            self.layers.append(subs)

    @staticmethod
    def _sublayer(w, pre, q, body):
        hc = f"{pre}hc{q}."
        f = lambda n: w[n].float().contiguous() if n in w else None   # noqa: E731  (a model without hyper-connection tensors has a plain residual)
        return _Sublayer(w[f"{pre}norm{q}"].float().contiguous(), f(hc + "in"), f(hc + "mix"), f(hc + "out"), body)

    def state_specs(self):
        """One entry per layer RUN (a layer that runs again has a cache and state of its own): what the state manager allocates."""
        return [self.layers[li][0].body.state_spec() for li in self.runs]

    def forward(self, step, ids, states, rows, n_rows, tap=None):
        """The step's tokens through every layer run; returns logits [n_rows][vocab] (fp32) of the batch rows listed in ``rows``."""
        ops, c, T, d, S = self.ops, self.cfg, step.T, self.width, self.streams
        x = step.scratch("streams", S * T * d)
        h = step.scratch("normed", T * d)
        y = step.scratch("sub_out", T * d)
        ops.embed(ids, self.embed, self.vocab, d, S, x, T, step.st)
        # the sublayers in the order they run; between two of them the write of the first and the read (+ norm) of the second are one kernel
        chain = [(r, k, sub) for r, li in enumerate(self.runs) for k, sub in enumerate(self.layers[li])]
        first = chain[0][2]
        ops.hyper_read(x, S, T, d, first.hc_in, first.norm_w, c.norm_groups, c.norm_eps, h, step.st)
        for i, (r, k, sub) in enumerate(chain):
            sub.body.forward(step, h, states[r], y)
            last_of_run = i + 1 == len(chain) or chain[i + 1][0] != r
            nxt = chain[i + 1][2] if i + 1 < len(chain) else None
            if tap is not None and last_of_run:          # inspection of the stream sum after a layer run: the unfused kernels
                ops.hyper_write(x, S, T, d, sub.hc_mix, sub.hc_out, y, step.st)
                ops.hyper_read(x, S, T, d, None, None, 1, 0.0, h, step.st)
                tap(r, h[:T * d].view(T, d))
                if nxt is not None:
                    ops.hyper_read(x, S, T, d, nxt.hc_in, nxt.norm_w, c.norm_groups, c.norm_eps, h, step.st)
                elif n_rows:
                    ops.hyper_read(x, S, T, d, None, self.final_norm, c.norm_groups, c.norm_eps, h, step.st)
            elif nxt is not None:
                ops.hyper_write_read(x, S, T, d, sub.hc_mix, sub.hc_out, y, nxt.hc_in, nxt.norm_w, c.norm_groups, c.norm_eps, h, step.st)
            elif n_rows:                                 # after the last sublayer: the sum of the streams through the model's norm
                ops.hyper_write_read(x, S, T, d, sub.hc_mix, sub.hc_out, y, None, self.final_norm, c.norm_groups, c.norm_eps, h, step.st)
            else:
                ops.hyper_write(x, S, T, d, sub.hc_mix, sub.hc_out, y, step.st)
        if n_rows == 0:
            return None
        picked = step.scratch("picked", n_rows * d)
        ops.gather_rows(h, d, rows, n_rows, d, picked, step.st)
        logits = step.scratch("logits", n_rows * self.vocab)
        T_save = step.T
        step.T = n_rows               # the head runs over the picked rows only
        try:
            self.head(step, picked.data_ptr(), d, logits.data_ptr(), self.vocab)
        finally:
            step.T = T_save
        return logits[:n_rows * self.vocab].view(n_rows, self.vocab)
