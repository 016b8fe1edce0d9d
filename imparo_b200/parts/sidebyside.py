"""Several mixers that read the same input, as one mixer (mixer "side_by_side").

Each branch is a mixer of its own (its own tensors under its own prefix, its own cache needs).  The result is the
mean of the branches' outputs, each first RMS-normed over the model width with a plain weight of its own:

    out = (1 / n) * sum_b  rms(branch_b(x)) * w_b

added into the stream times `scale` (the arrangement's residual factor).  The branches write 32-bit buffers
[tokens, hidden]; the norms, the mean and the add are one kernel.

With `weights` (a factor per branch) the result is instead the plain weighted sum  out = sum_b weights[b] * branch_b(x),
without norms (no norm tensors are read); the sum and the add are one kernel.

Branches that all keep their first product in 32-bit (wide_input_rows() > 0: heads prepared in 32-bit, a recurrence that is
fed unrounded rows) get it from ONE 32-bit product over the stacked matrices, made here.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import Part, make_part
from .spec import WeightSpec


class SideBySideMixer(Part):
    """params: hidden, eps, branches: a sequence of (sub-prefix, PartSpec of a mixer, name of its output-norm weight
    after this part's prefix; None with `weights`), weights (optional: a factor per branch; the branches' outputs are then
    summed with these factors and not normed)."""
    takes_scale = True

    def __init__(self, params, prefix, rt):
        super().__init__(params, prefix, rt)
        self.hidden = int(params["hidden"])
        self.eps = float(params.get("eps", 0.0))
        self.weights = tuple(float(w) for w in params["weights"]) if params.get("weights") is not None else None
        self.branches = []
        for sub, spec, norm_name in params["branches"]:
            self.branches.append((make_part("mixer", spec, prefix + sub, rt), prefix + norm_name if norm_name else None))
        if self.weights is not None and len(self.weights) != len(self.branches):
            raise ValueError("side-by-side mixer: one weight per branch")
        if self.weights is None and any(n is None for _, n in self.branches):
            raise ValueError("side-by-side mixer: every branch needs its output-norm weight (or the mixer its `weights`)")
        if not 1 <= len(self.branches) <= 4:
            raise ValueError("side-by-side mixer: one to four branches")
        self.graph_safe = all(b.graph_safe for b, _ in self.branches)
        self.norm_w = []
        self._n_caches = [len(b.cache_specs()) for b, _ in self.branches]

    def weight_specs(self):
        specs = []
        for b, norm_name in self.branches:
            specs += b.weight_specs()
            if self.weights is None:
                specs.append(WeightSpec(norm_name, ((self.hidden,),), role="vector", init=("norm",)))
        return specs

    def bind(self, tensors):
        self.norm_w = []
        for b, norm_name in self.branches:
            b.bind(tensors)
            if self.weights is None:
                self.norm_w.append(tensors[norm_name])
        self._wide_w = None
        self._wide()                  # the stacked matrix is made now, not at a first step (which may be recorded as a graph)

    def cache_specs(self):
        return tuple(s for b, _ in self.branches for s in b.cache_specs())

    # the branches' first products as one (see Part.input_rows): columns in the branches' order, each branch's range
    # starting at a multiple of 8 columns (16-byte rows for the consumers' vector loads)
    def _ranges(self):
        out, at = [], 0
        for b, _ in self.branches:
            n = b.input_rows()
            at = (at + 7) // 8 * 8
            out.append((at, n))
            at += n
        return out, at

    def input_rows(self) -> int:
        if any(b.input_rows() == 0 for b, _ in self.branches):
            return 0
        return self._ranges()[1]

    def input_weight(self):
        ranges, total = self._ranges()
        first = self.branches[0][0].input_weight()
        w = torch.zeros((total, first.shape[1]), dtype=first.dtype, device=first.device)
        for (b, _), (at, n) in zip(self.branches, ranges):
            w[at:at + n] = b.input_weight()
        return w

    def adopt_input_weight(self, view) -> None:
        for (b, _), (at, n) in zip(self.branches, self._ranges()[0]):
            b.adopt_input_weight(view[at:at + n])

    def _wide(self):
        """(stacked matrix, column ranges) of the branches' 32-bit first products, when every branch has one."""
        if getattr(self, "_wide_w", None) is None:
            self._wide_w = False
            subs = [b for b, _ in self.branches]
            if len(subs) > 1 and all(getattr(b, "wide_input_rows", lambda: 0)() > 0 for b in subs):
                ranges, at = [], 0
                for b in subs:
                    at = (at + 3) // 4 * 4
                    ranges.append((at, b.wide_input_rows()))
                    at += b.wide_input_rows()
                first = subs[0].wide_input_weight()
                w = torch.zeros((at, first.shape[1]), dtype=first.dtype, device=first.device)
                for b, (a, n) in zip(subs, ranges):
                    w[a:a + n] = b.wide_input_weight()
                    b.adopt_wide_input_weight(w[a:a + n])
                self._wide_w = (w, ranges)
        return self._wide_w

    def forward(self, x, batch, caches, residual, scale: float = 1.0, extra=None, extra_scale: float = 0.0, projected=None):
        """extra: a float32 [tokens, hidden] buffer added as well, times extra_scale, in the same pass over the
        stream (the arrangement's other sublayer).  projected: the branches' first products, made by the arrangement."""
        rt, T = self.rt, x.shape[0]
        outs, at = [], 0
        ranges = self._ranges()[0] if projected is not None else None
        wide = self._wide() if projected is None else False
        if wide:
            w, ranges = wide
            projected = rt.workspace.get("branches_in32", (T, w.shape[0]), torch.float32, first="tokens")
            ops.linear(x, w, projected, status=rt.status)
        for i, (b, _) in enumerate(self.branches):
            buf = rt.workspace.get(f"branch_out_{i}", (T, self.hidden), torch.float32, first="tokens")
            kw = {} if projected is None else {"projected": projected[:, ranges[i][0]:ranges[i][0] + ranges[i][1]]}
            b.forward(x, batch, caches[at:at + self._n_caches[i]], buf, accumulate=False, **kw)
            at += self._n_caches[i]
            outs.append(buf)
        if self.weights is not None:
            ys, cs = list(outs), [scale * w for w in self.weights]
            if extra is not None:
                ys.append(extra)
                cs.append(extra_scale)
            ops.add_weighted(residual, ys[:4], cs[:4])
            if len(ys) > 4:
                ops.add_weighted(residual, ys[4:], cs[4:])
            return
        # (the add may stay pending for the next norm of the stream to carry out: ops.allow_deferred_add by the arrangement)
        ops.norm_mean_add(residual, outs, self.norm_w, self.eps, scale / len(outs), extra, extra_scale, defer=True)
