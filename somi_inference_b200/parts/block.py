"""How a layer's parts are arranged around the residual stream.

Pre-norm (somi_inference/models/qwen2.py:325-339):
    x = x + mixer(norm1(x));  x = x + feed_forward(norm2(x)).
The residual stream `x` is float32 and the sums are made in float32, inside the
norm kernel: a block receives the previous block's output as `pending`, adds it
while normalising, and returns its own feed-forward output as the next `pending`.
"""

from __future__ import annotations

from .base import BranchSum, GatedDelta, NormedDelta, ScaledBranches, StateNeeds
from .registry import ARRANGEMENTS


@ARRANGEMENTS.register("pre_norm")
class PreNormBlock:
    def __init__(self, mixer, feed_forward, norms) -> None:
        if mixer is None or feed_forward is None:
            raise ValueError("the pre-norm arrangement needs a mixer and a feed-forward")
        if set(norms) != {"mixer", "feed_forward"}:
            raise ValueError("the pre-norm arrangement takes the norms 'mixer' and "
                             f"'feed_forward', got {sorted(norms)}")
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.mixer_norm = norms["mixer"]
        self.feed_forward_norm = norms["feed_forward"]

    def forward(self, residual, pending, batch, cache, owns_cache):
        h = self.mixer_norm.forward(residual, pending)
        a = self.mixer.forward(h, batch, cache, owns_cache)
        h = self.feed_forward_norm.forward(residual, a)
        return self.feed_forward.forward(h, batch)


@ARRANGEMENTS.register("sandwich_norm")
class SandwichNormBlock:
    """A norm before and a norm behind each branch:
        x = x + norm_b(mixer(norm_a(x)));  x = x + norm_d(feed_forward(norm_c(x)))
    Norms: `mixer`, `mixer_post`, and with a feed-forward `feed_forward`, `feed_forward_post`.  The
    post norms must be RMS norms: their weight and eps travel with the branch's result as a
    `NormedDelta`, and the next norm's kernel normalises the branch, adds it to the residual
    stream and normalises that, all in float32."""

    def __init__(self, mixer, feed_forward, norms) -> None:
        if mixer is None:
            raise ValueError("the sandwich arrangement needs a mixer")
        want = {"mixer", "mixer_post"}
        if feed_forward is not None:
            want |= {"feed_forward", "feed_forward_post"}
        if set(norms) != want:
            raise ValueError(f"the sandwich arrangement takes the norms {sorted(want)}, "
                             f"got {sorted(norms)}")
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.mixer_norm = norms["mixer"]
        self.mixer_post = norms["mixer_post"]
        self.feed_forward_norm = norms.get("feed_forward")
        self.feed_forward_post = norms.get("feed_forward_post")

    def forward(self, residual, pending, batch, cache, owns_cache):
        h = self.mixer_norm.forward(residual, pending)
        a = self.mixer.forward(h, batch, cache, owns_cache)
        pending = NormedDelta(a, self.mixer_post.weight, self.mixer_post.eps)
        if self.feed_forward is None:
            return pending
        h = self.feed_forward_norm.forward(residual, pending)
        f = self.feed_forward.forward(h, batch)
        return NormedDelta(f, self.feed_forward_post.weight, self.feed_forward_post.eps)


@ARRANGEMENTS.register("gated_pre_norm")
class GatedPreNormBlock:
    """Pre-norm with a gate on each branch and a short convolution in front of the mixer:
        h = norm1(x);  x = x + sigmoid(G1 h) * mixer(h + conv(h))
        h = norm2(x);  x = x + sigmoid(G2 h) * feed_forward(h)          (where the layer has one)
    The gates read what the norm produced (before the convolution).  Extras: `mixer_gate`,
    `mixer_taps` (either may be absent), `feed_forward_gate`.  The sums and the sigmoid are made
    by the next norm's kernel, which gets the branch and the gate's logits as a `GatedDelta`."""

    def __init__(self, mixer, feed_forward, norms, extras=None) -> None:
        extras = dict(extras or {})
        if mixer is None:
            raise ValueError("the gated pre-norm arrangement needs a mixer")
        want = {"mixer"} | ({"feed_forward"} if feed_forward is not None else set())
        if set(norms) != want:
            raise ValueError(f"the gated pre-norm arrangement takes the norms {sorted(want)}, "
                             f"got {sorted(norms)}")
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.mixer_norm = norms["mixer"]
        self.feed_forward_norm = norms.get("feed_forward")
        self.mixer_gate = extras.pop("mixer_gate", None)
        self.mixer_taps = extras.pop("mixer_taps", None)
        self.feed_forward_gate = extras.pop("feed_forward_gate", None)
        if extras:
            raise ValueError(f"the gated pre-norm arrangement has no use for {sorted(extras)}")
        # the feed-forward's gate reads the same rows as its up projection: one product for both
        self.fused_ff_gate = (self.feed_forward_gate is not None
                              and hasattr(feed_forward, "attach_side"))
        if self.fused_ff_gate:
            feed_forward.attach_side(self.feed_forward_gate.weight, self.feed_forward_gate.bias)

    def state_needs(self) -> StateNeeds:
        return self.mixer_taps.state_needs() if self.mixer_taps is not None else StateNeeds({})

    def forward(self, residual, pending, batch, cache, owns_cache):
        h = self.mixer_norm.forward(residual, pending)
        gate = self.mixer_gate.logits(h) if self.mixer_gate is not None else None
        if self.mixer_taps is not None:
            h = self.mixer_taps.forward(h, batch, cache.state)
        pending = GatedDelta(self.mixer.forward(h, batch, cache, owns_cache), gate)
        if self.feed_forward is None:
            return pending
        h = self.feed_forward_norm.forward(residual, pending)
        if self.fused_ff_gate:
            y, gate = self.feed_forward.forward(h, batch, side=True)
            return GatedDelta(y, gate)
        gate = self.feed_forward_gate.logits(h) if self.feed_forward_gate is not None else None
        return GatedDelta(self.feed_forward.forward(h, batch), gate)


@ARRANGEMENTS.register("parallel_branches")
class ParallelBranchesBlock:
    """Mixer and feed-forward read the same stream, each through a norm of its own:
        x = x + mult * (scale_m * mixer(norm_m(x)) + scale_f * feed_forward(norm_f(x)))
    `scale_m`, `scale_f`: per-channel scales (layer extras `mixer_scale`, `feed_forward_scale`;
    either may be absent), `mult` the factor of extra `branch_factor` (absent: 1).  A layer
    without a feed-forward has the mixer's branch only.  Norms: `mixer`, and with a feed-forward
    `feed_forward`; both must be RMS norms: one kernel adds what the layer before left (a
    `ScaledBranches`), writes the stream and produces both normalised rows from it in float32."""

    def __init__(self, mixer, feed_forward, norms, extras=None) -> None:
        extras = dict(extras or {})
        if mixer is None:
            raise ValueError("the parallel-branches arrangement needs a mixer")
        want = {"mixer"} | ({"feed_forward"} if feed_forward is not None else set())
        if set(norms) != want:
            raise ValueError(f"the parallel-branches arrangement takes the norms {sorted(want)}, "
                             f"got {sorted(norms)}")
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.mixer_norm = norms["mixer"]
        self.feed_forward_norm = norms.get("feed_forward")
        if self.feed_forward_norm is not None and self.feed_forward_norm.eps != self.mixer_norm.eps:
            raise ValueError("the two norms of a parallel-branches layer share one eps")
        scale_m = extras.pop("mixer_scale", None)
        scale_f = extras.pop("feed_forward_scale", None)
        factor = extras.pop("branch_factor", None)
        if extras:
            raise ValueError(f"the parallel-branches arrangement has no use for {sorted(extras)}")
        self.mixer_scale = None if scale_m is None else scale_m.weight
        self.feed_forward_scale = None if scale_f is None else scale_f.weight
        self.mult = 1.0 if factor is None else factor.value

    def forward(self, residual, pending, batch, cache, owns_cache):
        hm, hf = self.mixer_norm.forward_pair(residual, pending, self.feed_forward_norm)
        a = self.mixer.forward(hm, batch, cache, owns_cache)
        f = None if self.feed_forward is None else self.feed_forward.forward(hf, batch)
        return ScaledBranches(a, self.mixer_scale, f,
                              None if f is None else self.feed_forward_scale, self.mult)


@ARRANGEMENTS.register("shared_norm")
class SharedNormBlock:
    """Mixer and feed-forward read the output of one norm, and both results join the stream:
        h = norm(x);  x = x + mixer(h) + feed_forward(h)
    A layer without a feed-forward has the mixer's branch only.  Norm: `shared`, of any kind whose
    `forward` takes a `BranchSum`: the sums are made in float32 by the next norm's kernel."""

    def __init__(self, mixer, feed_forward, norms) -> None:
        if mixer is None:
            raise ValueError("the shared-norm arrangement needs a mixer")
        if set(norms) != {"shared"}:
            raise ValueError(f"the shared-norm arrangement takes the norm 'shared', got {sorted(norms)}")
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.norm = norms["shared"]

    def forward(self, residual, pending, batch, cache, owns_cache):
        h = self.norm.forward(residual, pending)
        a = self.mixer.forward(h, batch, cache, owns_cache)
        f = None if self.feed_forward is None else self.feed_forward.forward(h, batch)
        return BranchSum(a, f)
