"""How a layer's parts are arranged.  "prenorm_residual" is the reference's block:
x += mixer(norm(x)); x += feed_forward(norm(x)), pre-norms only
(imparo-model/src/lfm2/workflow_cpu.rs:8-18,172-319)."""
from __future__ import annotations

from .base import Block, make_part


class PreNormResidualBlock(Block):
    """params: layer (LayerSpec)."""

    def __init__(self, params, prefix, rt):
        super().__init__(params, prefix, rt)
        spec = params["layer"]
        self.mixer_norm = make_part("norm", spec.mixer_norm, prefix, rt)
        self.mixer = make_part("mixer", spec.mixer, prefix, rt)
        self.ff_norm = make_part("norm", spec.feed_forward_norm, prefix, rt)
        self.ff = make_part("feed_forward", spec.feed_forward, prefix, rt)
        self.parts = (self.mixer_norm, self.mixer, self.ff_norm, self.ff)
        self.graph_safe = all(p.graph_safe for p in self.parts)
        self.picks_rows = True         # forward(only_rows=...) is implemented

    def weight_specs(self):
        return [w for p in self.parts for w in p.weight_specs()]

    def bind(self, tensors):
        for p in self.parts:
            p.bind(tensors)

    def cache_specs(self):
        return self.mixer.cache_specs()

    def forward(self, x, batch, caches, only_rows=None):
        """x: the 32-bit residual stream [tokens, width], updated in place.
        only_rows = (rows, n): the caller needs the block's output at these n rows only (the
        model's last block, whose output feeds nothing but the wanted logits; the reference skips
        the same work, imparo-model/src/lfm2/workflow_gpu.rs:990-992,1201-1203).  The mixer still
        runs on every row (its cache and state advance); the feed-forward runs on the picked rows,
        and their stream [n, width] is returned instead (None when n is 0)."""
        from ..kernels import ops
        if self.rt.probe_now:
            return self._forward_probed(x, batch, caches, only_rows)
        h = self.mixer_norm.forward(x, tag="normed_mixer")
        self._run(self.mixer, x, lambda: self.mixer.forward(h, batch, caches, x))
        if only_rows is not None:
            rows, n = only_rows
            if n == 0:
                ops.settle(x)
                return None
            xs = self.rt.workspace.get("stream_picked", (n, x.shape[1]), x.dtype, first="rows")
            ops.gather_rows(x, rows, xs)
            picked_in = self.ff_norm.forward(xs, tag="normed_ff")
            self._run(self.ff, xs, lambda: self.ff.forward(picked_in, batch, xs))
            return xs
        ff_in = self.ff_norm.forward(x, tag="normed_ff")
        self._run(self.ff, x, lambda: self.ff.forward(ff_in, batch, x))
        return None

    def _forward_probed(self, x, batch, caches, only_rows):
        """The same block with every stage evaluated and shown to the runtime's probe: the stream
        going in, the mixer's normed input, the stream after the mixer, the feed-forward's normed
        input, the stream going out.  Nothing is deferred here."""
        from ..kernels import ops
        probe = self.rt.probe
        ops.settle(x)
        probe("stream_in", x)
        h = self.mixer_norm.forward(x, tag="normed_mixer")
        probe("mixer_norm", h)
        ops.settle(x)
        self.mixer.forward(h, batch, caches, x)
        ops.settle(x)
        probe("stream_mixer", x)
        if only_rows is not None:
            rows, n = only_rows
            if n == 0:
                return None
            xs = self.rt.workspace.get("stream_picked", (n, x.shape[1]), x.dtype, first="rows")
            ops.gather_rows(x, rows, xs)
            x = xs
        ff_in = self.ff_norm.forward(x, tag="normed_ff")
        probe("ff_norm", ff_in)
        self.ff.forward(ff_in, batch, x)
        ops.settle(x)
        probe("stream_out", x)
        return x if only_rows is not None else None

    @staticmethod
    def _run(part, x, call) -> None:
        """A part whose last write to the stream is an accumulate-product may leave that add as
        split partials for the next norm to fold (ops.allow_deferred_add); any other part gets
        and leaves a stream that is whole."""
        from ..kernels import ops
        if part.adds_with_linear:
            ops.allow_deferred_add(x)
            try:
                call()
            finally:
                ops.disallow_deferred_add(x)
        else:
            ops.settle(x)
            call()


class ParallelResidualBlock(Block):
    """One norm, both sublayers read its output, one add:  h = norm(x);  x += s * (mixer(h) + feed_forward(h)).

    params: layer (LayerSpec).  The layer's mixer_norm is the one norm; feed_forward may be None (the layer has none);
    layer.params["residual_scale"] is s (default 1).  A mixer or feed-forward that is to be scaled declares
    takes_scale (its forward has a `scale` keyword).  When the mixer can take the other sublayer's output along
    (forward(..., extra=, extra_scale=), as the side-by-side mixer does) and the feed-forward can write into a
    buffer (forward_into), the feed-forward runs first and both are added in the mixer's one pass over the stream."""

    def __init__(self, params, prefix, rt):
        super().__init__(params, prefix, rt)
        spec = params["layer"]
        self.scale = float(spec.params.get("residual_scale", 1.0))
        self.norm = make_part("norm", spec.mixer_norm, prefix, rt)
        self.mixer = make_part("mixer", spec.mixer, prefix, rt)
        self.ff = make_part("feed_forward", spec.feed_forward, prefix, rt) if spec.feed_forward is not None else None
        self.parts = tuple(p for p in (self.norm, self.mixer, self.ff) if p is not None)
        for p in self.parts[1:]:
            if self.scale != 1.0 and not getattr(p, "takes_scale", False):
                raise ValueError(f"parallel block: {type(p).__name__} cannot scale its output (residual_scale {self.scale})")
        self.graph_safe = all(p.graph_safe for p in self.parts)
        self.picks_rows = False
        import inspect
        self._one_pass = (self.ff is not None and hasattr(self.ff, "forward_into")
                          and "extra" in inspect.signature(self.mixer.forward).parameters)
        # a feed-forward whose forward() has an `accumulate` keyword may default to overwriting: here it adds, or (beside
        # a mixer that takes the other sublayer's output along) writes a buffer that the mixer's one add carries in
        self._ff_adds = self.ff is not None and "accumulate" in inspect.signature(self.ff.forward).parameters
        self._ff_rides = (self._ff_adds and not self._one_pass
                          and "extra" in inspect.signature(self.mixer.forward).parameters)

    def weight_specs(self):
        return [w for p in self.parts for w in p.weight_specs()]

    def bind(self, tensors):
        import inspect
        import torch
        for p in self.parts:
            p.bind(tensors)
        # One product for everything that reads the normed input (Part.input_rows): the mixer's first products and the
        # feed-forward's, stacked; the parts keep views into the stacked matrix, so the weights exist once.
        self.w_in, self._in_ranges = None, None
        subs = [p for p in (self.mixer, self.ff) if p is not None]
        takes = "projected" in inspect.signature(self.mixer.forward).parameters
        if takes and all(p.input_rows() > 0 for p in subs) and (self.ff is None or self._one_pass):
            ranges, at = [], 0
            for p in subs:
                at = (at + 7) // 8 * 8
                ranges.append((at, p.input_rows()))
                at += p.input_rows()
            first = subs[0].input_weight()
            w = torch.zeros((at, first.shape[1]), dtype=first.dtype, device=first.device)
            for p, (a, n) in zip(subs, ranges):
                w[a:a + n] = p.input_weight()
                p.adopt_input_weight(w[a:a + n])
            self.w_in, self._in_ranges = w, ranges

    def cache_specs(self):
        return self.mixer.cache_specs()

    def forward(self, x, batch, caches, only_rows=None):
        from ..kernels import ops
        import torch
        probe = self.rt.probe if self.rt.probe_now else None
        if probe:
            ops.settle(x)
            probe("stream_in", x)
        h = self.norm.forward(x, tag="normed_mixer")          # (carries out an add the block before left pending)
        if probe:
            probe("mixer_norm", h)
        kw = {"scale": self.scale} if self.scale != 1.0 else {}
        if self.w_in is not None and not probe:
            both = self.rt.workspace.get("block_in", (x.shape[0], self.w_in.shape[0]), self.rt.act_dtype, first="tokens")
            ops.linear(h, self.w_in, both, status=self.rt.status)
            ma, mn = self._in_ranges[0]
            kw["projected"] = both[:, ma:ma + mn]
        if self._one_pass and not probe:
            y = self.rt.workspace.get("ffn_out", (x.shape[0], x.shape[1]), torch.float32, first="tokens")
            if self.w_in is not None:
                fa, fn = self._in_ranges[1]
                self.ff.forward_into(h, y, projected=both[:, fa:fa + fn])
            else:
                self.ff.forward_into(h, y)
            # the mixer's add is the block's last write to the stream: it may stay pending for the next norm
            ops.allow_deferred_add(x)
            try:
                self.mixer.forward(h, batch, caches, x, extra=y, extra_scale=self.scale, **kw)
            finally:
                ops.disallow_deferred_add(x)
            return None
        if self._ff_rides and not probe:
            y = self.rt.workspace.get("ffn_out", (x.shape[0], x.shape[1]), torch.float32, first="tokens")
            self.ff.forward(h, batch, y, accumulate=False)
            self.mixer.forward(h, batch, caches, x, extra=y, extra_scale=self.scale, **kw)
            return None
        self.mixer.forward(h, batch, caches, x, **kw)
        kw.pop("projected", None)
        ops.settle(x)
        if probe:
            probe("stream_mixer", x)
        if self.ff is not None:
            if self._ff_adds:
                kw["accumulate"] = True
            self.ff.forward(h, batch, x, **kw)
        ops.settle(x)
        if probe:
            probe("stream_out", x)
        return None


class OutputNormResidualBlock(Block):
    """The norm sits on each sublayer's OUTPUT only:  x += norm1(mixer(x));  x += norm2(feed_forward(x)).

    params: layer (LayerSpec): mixer_norm is norm1, feed_forward_norm norm2 (both "rmsnorm" parts; their weight and eps
    are what the add kernel applies); feed_forward may be None.  The sublayers read the stream itself: in 32-bit the
    stream, in bfloat16 its rounding, which the add kernel of the sublayer before stores beside the updated stream
    (batch.notes["stream_copy"]; the first block of a step makes it with a cast).  Sublayers write their output into a
    float32 buffer (forward(..., accumulate=False)); one kernel norms it and adds it into the stream."""

    def __init__(self, params, prefix, rt):
        super().__init__(params, prefix, rt)
        spec = params["layer"]
        self.mixer_norm = make_part("norm", spec.mixer_norm, prefix, rt)
        self.mixer = make_part("mixer", spec.mixer, prefix, rt)
        self.ff = make_part("feed_forward", spec.feed_forward, prefix, rt) if spec.feed_forward is not None else None
        self.ff_norm = make_part("norm", spec.feed_forward_norm, prefix, rt) if self.ff is not None else None
        self.parts = tuple(p for p in (self.mixer_norm, self.mixer, self.ff_norm, self.ff) if p is not None)
        self.graph_safe = all(p.graph_safe for p in self.parts)
        self.picks_rows = True

    def weight_specs(self):
        return [w for p in self.parts for w in p.weight_specs()]

    def bind(self, tensors):
        for p in self.parts:
            p.bind(tensors)

    def cache_specs(self):
        return self.mixer.cache_specs()

    def _input(self, x, batch, tag="stream_copy"):
        """What the sublayer's products read: the stream (32-bit path) or its copy in the activation dtype."""
        import torch
        from ..kernels import ops
        if self.rt.act_dtype == torch.float32:
            return x
        notes = getattr(batch, "notes", None)
        if notes is not None and notes.get("stream_copy_of") == x.data_ptr():
            return notes["stream_copy"]
        h = self.rt.workspace.get(tag, tuple(x.shape), self.rt.act_dtype, first="tokens" if tag == "stream_copy" else "rows")
        ops.cast_rows(x, h)
        return h

    def _add(self, x, y, norm, batch, tag="stream_copy"):
        """x += norm(y); in bfloat16 the updated rows are also left as the next sublayer's input."""
        import torch
        from ..kernels import ops
        copy = None
        if self.rt.act_dtype != torch.float32:
            copy = self.rt.workspace.get(tag, tuple(x.shape), self.rt.act_dtype, first="tokens" if tag == "stream_copy" else "rows")
        ops.out_norm_add(x, y, norm.weight, norm.eps, copy=copy)
        notes = getattr(batch, "notes", None)
        if copy is not None and notes is not None and tag == "stream_copy":
            notes["stream_copy"], notes["stream_copy_of"] = copy, x.data_ptr()
        return copy if copy is not None else x

    def forward(self, x, batch, caches, only_rows=None):
        import torch
        from ..kernels import ops
        probe = self.rt.probe if self.rt.probe_now else None
        ws = self.rt.workspace
        ops.settle(x)
        if probe:
            probe("stream_in", x)
        y = ws.get("sublayer_out", tuple(x.shape), torch.float32, first="tokens")
        self.mixer.forward(self._input(x, batch), batch, caches, y, accumulate=False)
        ops.settle(y)
        h = self._add(x, y, self.mixer_norm, batch)
        if probe:
            probe("stream_mixer", x)
        if only_rows is not None:
            rows, n = only_rows
            if n == 0:
                return None
            xs = ws.get("stream_picked", (n, x.shape[1]), x.dtype, first="rows")
            ops.gather_rows(x, rows, xs)
            if self.ff is not None:
                ys = ws.get("sublayer_out_picked", (n, x.shape[1]), torch.float32, first="rows")
                self.ff.forward(self._input(xs, None, tag="stream_copy_picked"), batch, ys, accumulate=False)
                ops.settle(ys)
                self._add(xs, ys, self.ff_norm, None, tag="stream_copy_picked")
            if probe:
                probe("stream_out", xs)
            return xs
        if self.ff is not None:
            self.ff.forward(h, batch, y, accumulate=False)
            ops.settle(y)
            self._add(x, y, self.ff_norm, batch)
        if probe:
            probe("stream_out", x)
        return None


class HyperConnectionBlock(Block):
    """The stream is kept as n copies per token, x [tokens, n * width] ("hyper-connections").  For each sublayer f (the
    mixer, then the feed-forward if the layer has one) with its own tensors a [n], b [n], M [n, n] (indexed [from, to]):

        u = sum_s a[s] x_s;   y = f(norm(u));   x_t <- sum_s M[s, t] x_s + b[t] y      (all copies at once from the old ones)

    params: layer (LayerSpec): mixer_norm / feed_forward_norm are "rmsnorm" parts with `streams` = n and `stream_weights` =
    the name of a; layer.params: "streams" (n), "mixer_hc" and "feed_forward_hc" ({"out": name of b, "mix": name of M}).
    Sublayers write their output into a float32 buffer (forward(..., accumulate=False)).  The update of the copies is left
    to the next reader of the stream: the next sublayer's norm (of this block or of the one after it) mixes, adds and norms
    in one pass.  As the model's last block the feed-forward runs on the wanted rows only.  Without "mixer_hc" /
    "feed_forward_hc" no tensors are read and b and M are ones: with n = 1 that is the plain pre-norm block
    x <- x + f(norm(x)), for layers with or without a feed-forward."""

    def __init__(self, params, prefix, rt):
        super().__init__(params, prefix, rt)
        spec = params["layer"]
        self.n = int(spec.params["streams"])
        self.mixer_norm = make_part("norm", spec.mixer_norm, prefix, rt)
        self.mixer = make_part("mixer", spec.mixer, prefix, rt)
        self.ff = make_part("feed_forward", spec.feed_forward, prefix, rt) if spec.feed_forward is not None else None
        self.ff_norm = make_part("norm", spec.feed_forward_norm, prefix, rt) if self.ff is not None else None
        names = [spec.params.get("mixer_hc")] + ([spec.params.get("feed_forward_hc")] if self.ff is not None else [])
        self.hc_names = [dict(x) if x else None for x in names]
        if any(x is None for x in self.hc_names) and self.n != 1:
            raise ValueError("hyper-connection block: several copies of the stream need their mixing tensors")
        self.parts = tuple(p for p in (self.mixer_norm, self.mixer, self.ff_norm, self.ff) if p is not None)
        self.graph_safe = all(p.graph_safe for p in self.parts)
        self.picks_rows = True
        self.hc = []

    def weight_specs(self):
        from .spec import WeightSpec
        n = self.n
        specs = [w for p in self.parts for w in p.weight_specs()]
        for names in self.hc_names:
            if names is not None:
                specs += [WeightSpec(self.prefix + names["out"], ((n,),), role="vector", init=("uniform", 0.5, 1.0)),
                          WeightSpec(self.prefix + names["mix"], ((n, n),), role="vector", init=("uniform", 0.0, 0.6))]
        return specs

    def bind(self, tensors):
        for p in self.parts:
            p.bind(tensors)
        import torch
        one = torch.ones(1, dtype=torch.float32, device=self.rt.device)
        self.hc = [(one, one) if names is None else (tensors[self.prefix + names["mix"]].contiguous(), tensors[self.prefix + names["out"]])
                   for names in self.hc_names]

    def cache_specs(self):
        return self.mixer.cache_specs()

    def forward(self, x, batch, caches, only_rows=None):
        import torch
        from ..kernels import ops
        probe = self.rt.probe if self.rt.probe_now else None
        ws = self.rt.workspace
        width = x.shape[1] // self.n
        if probe:
            ops.settle(x)
            probe("stream_in", x)
        h = self.mixer_norm.forward(x, tag="normed_mixer")           # (carries out the update the sublayer before left pending)
        if probe:
            probe("mixer_norm", h)
        y = ws.get("sublayer_out", (x.shape[0], width), torch.float32, first="tokens")
        self.mixer.forward(h, batch, caches, y, accumulate=False)
        mix, out = self.hc[0]
        ops.streams_mix_add(x, self.n, mix, out, y, defer=not probe)
        if probe:
            probe("stream_mixer", x)
        if only_rows is not None:
            rows, n = only_rows
            if n == 0:
                ops.settle(x)
                return None
            xs = ws.get("stream_picked", (n, x.shape[1]), x.dtype, first="rows")
            ops.gather_rows(x, rows, xs)
            if self.ff is not None:
                hs = self.ff_norm.forward(xs, tag="normed_ff_picked")
                ys = ws.get("sublayer_out_picked", (n, width), torch.float32, first="rows")
                self.ff.forward(hs, batch, ys, accumulate=False)
                mix, out = self.hc[1]
                ops.streams_mix_add(xs, self.n, mix, out, ys)
            if probe:
                probe("stream_out", xs)
            return xs
        if self.ff is not None:
            h = self.ff_norm.forward(x, tag="normed_ff")
            if probe:
                probe("ff_norm", h)
            self.ff.forward(h, batch, y, accumulate=False)
            mix, out = self.hc[1]
            ops.streams_mix_add(x, self.n, mix, out, y, defer=not probe)
        if probe:
            probe("stream_out", x)
        return None
