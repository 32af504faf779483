"""Sopetar: a decoder-only model of parallel layers — ONE layer norm (weight and bias) feeds a sequence mixer and a feed-forward whose
results are both added to the layer's input — with a depth-weighted average between layers: what a layer passes on is a learned
combination of the embedding output and of every layer's own result so far. The mixers are softmax attention without rotation (unit-rms
heads, capped scores, distance slopes, a sliding window that keeps the first positions, values blended with those of the first such
layer) and latent attention (one cached latent row per token, a rotated key part shared by the heads, a softmax sink, a head gate).

The class only DESCRIBES the model with the mechanisms of ``layers``; cache, batching and the step loop belong to
``seqengine.SequenceEngine``. Tensor names: ``embed``, ``l<i>.norm1`` (+ ``.b``), ``l<i>.mix.*``, ``l<i>.mlp.*``, ``l<i>.dwa``,
``final.norm`` (+ ``.b``), ``head``."""
from __future__ import annotations

from ..layers import CappedWindowAttention, ClampedGluFeedForward, FusedLinear, LatentAttention, MixerGroup


class _Layer:
    def __init__(self, norm_w, norm_b, group, depth_coef):
        self.norm_w, self.norm_b, self.group, self.depth_coef = norm_w, norm_b, group, depth_coef


class SopetarModel:
    def __init__(self, cfg, w, ops, device):
        self.cfg, self.ops, self.device = cfg, ops, device
        self.vocab, self.width = cfg.vocab, cfg.width
        f = lambda n: w[n].float().contiguous()   # noqa: E731
        self.embed = w["embed"].contiguous()
        self.final_w, self.final_b = f("final.norm"), f("final.norm.b")
        self.head = FusedLinear([(w["head"], None)], ops, device)
        self.layers = []
        first_shared = None
        for i, lc in enumerate(cfg.layers):
            pre = f"l{i}."
            if lc.type == "attention":
                share = None
                if lc.mixer.v_mix:
                    share = "keep" if first_shared is None else "blend"
                    first_shared = i if first_shared is None else first_shared
                mixer = CappedWindowAttention(lc.mixer, w, pre + "mix.", ops, device, cfg.norm_eps, share)
            else:
                mixer = LatentAttention(lc.mixer, w, pre + "mix.", ops, device, cfg.norm_eps)
            members = [("mix", mixer, 1.0)]
            if lc.mlp is not None:
                members.append(("ff", ClampedGluFeedForward(lc.mlp, w, pre + "mlp.", ops, device), 1.0))
            coef = f(pre + "dwa")
            if coef.numel() != i + 2:
                raise ValueError(f"{pre}dwa holds {coef.numel()} coefficients, layer {i} combines {i + 2} results")
            self.layers.append(_Layer(f(pre + "norm1"), f(pre + "norm1.b"), MixerGroup(members, ops, device), coef))

    def state_specs(self):
        return [l.group.state_spec() for l in self.layers]

    def forward(self, step, ids, states, rows, n_rows, tap=None):
        """The step's tokens through every layer; returns logits [n_rows][vocab] (fp32) of the batch rows listed in ``rows``."""
        ops, c, T, d, L = self.ops, self.cfg, step.T, self.width, len(self.layers)
        # planes of [T][d]: the stream that the next layer reads, then the embedding output, then every layer's own result
        planes = step.scratch("depth_planes", (L + 2) * T * d)
        x, hist = planes[:T * d], planes[T * d:]
        h = step.scratch("normed", T * d)
        y = step.scratch("sub_out", T * d)
        ops.embed(ids, self.embed, self.vocab, d, 2, planes, T, step.st, scale=c.embedding_scale)   # layer 0 reads the embedding output itself
        first = self.layers[0]
        # a norm whose rows feed a tensor-core product also leaves them as that product's bf16 operand
        h16 = first.group.proj.operand_rows(step)
        ops.layernorm(x, d, first.norm_w, first.norm_b, c.norm_eps, h, d, T, d, step.st, y16=h16)
        for i, layer in enumerate(self.layers):
            layer.group.forward(step, h, states[i], y, h16_ready=h16 is not None)
            nxt = self.layers[i + 1] if i + 1 < L else None
            norm_w, norm_b = (nxt.norm_w, nxt.norm_b) if nxt is not None else ((self.final_w, self.final_b) if n_rows else (None, None))
            h16 = nxt.group.proj.operand_rows(step) if nxt is not None else None
            # the layer's own result, the weighted average over the depth, and the norm of what follows, as one kernel
            ops.depth_average(x, y, hist, i + 1, layer.depth_coef, norm_w, norm_b, c.norm_eps, h, T, d, step.st, h16=h16)
            if tap is not None:
                tap(i, x[:T * d].view(T, d))
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
