"""Parts, a block arrangement and a whole architecture of other kinds than the framework's own, defined in the tests:
a mixer with per-request state, a routed feed-forward, a position part without rotation, and a toy architecture that
puts them together, with a typed configuration read from its own config.json keys. Nothing in serve_b200 knows of them;
registering them here is all it takes. Both the CPU tests (with torch stand-ins for the kernels) and the GPU tests use them."""
import torch

from serve_b200.config import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from serve_b200.config.base import ConfigError, ModelConfig, register_architecture
from serve_b200.parts import CacheNeed, FeedForward, Mixer, PositionEncoding, TensorDecl, register_part
from tests.plain import llama_plain as P


# ---- parts of other kinds, defined here, never part of any model of the framework ----------------------
@register_part("mixer", "test_running_mean")
class RunningMeanMixer(Mixer):
    """A toy mixer with per-request state of fixed size: out_t = W * mean(h_0..h_t). State: sum [hidden] and count [1]."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.hidden = int(spec.params["hidden"])
        self.w = None

    def tensor_decls(self):
        return [TensorDecl(self.prefix + "mix.weight", (self.hidden, self.hidden))]

    def load(self, tensors):
        self.w = tensors[self.prefix + "mix.weight"]

    def cache_need(self):
        return CacheNeed(state_shape=(self.hidden + 1,))

    def forward(self, h, ctx, cache):
        if ctx.shape.pure_decode:
            # one token per request: device-side indexing only, so that the step can be captured in a graph
            slots = ctx.slots.long()
            st = cache.state[slots]
            sums = st[:, : self.hidden] + h.float()
            counts = st[:, self.hidden] + 1
            cache.state[slots] = torch.cat([sums, counts[:, None]], 1)
            return ((sums / counts[:, None]) @ self.w.float().T).to(h.dtype)
        out = torch.empty_like(h)
        cu = ctx.cu_q.tolist()
        for r, slot in enumerate(ctx.slots.tolist()):
            a, b = cu[r], cu[r + 1]
            st = cache.state[slot]
            sums = st[: self.hidden] + torch.cumsum(h[a:b].float(), 0)
            counts = st[self.hidden] + torch.arange(1, b - a + 1, device=h.device)
            out[a:b] = ((sums / counts[:, None]) @ self.w.float().T).to(h.dtype)
            st[: self.hidden] = sums[-1]
            st[self.hidden] = counts[-1]
        return out


@register_part("feed_forward", "test_top1_experts")
class Top1Experts(FeedForward):
    """A toy routed feed-forward: router logits in float32, the best expert's matrix is applied."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.hidden, self.experts = int(spec.params["hidden"]), int(spec.params["experts"])

    def tensor_decls(self):
        return [TensorDecl(self.prefix + "router.weight", (self.experts, self.hidden)),
                TensorDecl(self.prefix + "experts.weight", (self.experts * self.hidden, self.hidden))]

    def load(self, tensors):
        self.router = tensors[self.prefix + "router.weight"]
        self.w = tensors[self.prefix + "experts.weight"].view(self.experts, self.hidden, self.hidden)

    def forward(self, h, ctx):
        pick = (h.float() @ self.router.float().T).argmax(-1)
        return torch.einsum("th,tch->tc", h.float(), self.w.float()[pick]).to(h.dtype)


@register_part("position", "test_none_but_marker")
class MarkerPosition(PositionEncoding):
    """Another position encoding for the attention mixer: no rotation at all (rotary_dim 0)."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.rotary_dim, self.pairing = 0, 0
        self.inv_freq = torch.zeros(1, dtype=torch.float32, device=runtime.device)


def toy_spec(hidden, vocab):
    norm = lambda p: PartSpec("rms", {"size": hidden, "eps": 1e-5}, prefix=p)
    att = PartSpec("attention", {"hidden": hidden, "heads": 4, "kv_heads": 2, "head_dim": 16, "scale": None, "window": None,
                                 "position": PartSpec("test_none_but_marker", {})}, prefix="l1.att.")
    layers = [
        LayerSpec.pre_norm(PartSpec("test_running_mean", {"hidden": hidden}, prefix="l0."),
                  PartSpec("test_top1_experts", {"hidden": hidden, "experts": 3}, prefix="l0.moe."), norm("l0.n1."), norm("l0.n2.")),
        LayerSpec.pre_norm(att, PartSpec("swiglu", {"hidden": hidden, "intermediate": 96}, prefix="l1.mlp."), norm("l1.n1."), norm("l1.n2.")),
    ]
    return ModelSpec("ToyForTests", hidden, vocab, PartSpec("table", {"vocab": vocab, "hidden": hidden, "name": "emb.weight"}),
                     layers, [ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0)], norm("final."),
                     PartSpec("linear", {"vocab": vocab, "hidden": hidden, "name": "head.weight", "tied_to": "emb.weight"}), 512)


def toy_plain(w, tokens, hidden):
    """The same toy model, whole sequence, plain torch on the CPU."""
    x = w["emb.weight"][tokens]
    t = x.shape[0]
    def mean_mix(h):
        return (torch.cumsum(h, 0) / torch.arange(1, t + 1)[:, None]) @ w["l0.mix.weight"].T
    def moe(h):
        pick = (h @ w["l0.moe.router.weight"].T).argmax(-1)
        return torch.einsum("th,tch->tc", h, w["l0.moe.experts.weight"].view(3, hidden, hidden)[pick])
    def layer0(x):
        x = x + mean_mix(P.rms_norm(x, w["l0.n1.weight"], 1e-5))
        return x + moe(P.rms_norm(x, w["l0.n2.weight"], 1e-5))
    x = layer0(x)
    h = P.rms_norm(x, w["l1.n1.weight"], 1e-5)
    q = (h @ w["l1.att.q_proj.weight"].T).view(t, 4, 16)
    k = (h @ w["l1.att.k_proj.weight"].T).view(t, 2, 16)
    v = (h @ w["l1.att.v_proj.weight"].T).view(t, 2, 16)
    x = x + P.causal_attention(q, k, v, 0.25).reshape(t, 64) @ w["l1.att.o_proj.weight"].T
    x = x + P.swiglu(P.rms_norm(x, w["l1.n2.weight"], 1e-5), w["l1.mlp.gate_proj.weight"], w["l1.mlp.up_proj.weight"], w["l1.mlp.down_proj.weight"])
    x = layer0(x)
    return P.rms_norm(x, w["final.weight"], 1e-5) @ w["emb.weight"].T


# ---- a whole architecture of this kind: a configuration class for its own config.json keys, and its registration -----
from dataclasses import dataclass


@dataclass(frozen=True)
class ToyConfig(ModelConfig):
    width: int
    tokens: int
    longest: int = 512

    architecture = "ToyDecoderForTests"

    @classmethod
    def from_dict(cls, d):
        for key in ("width", "tokens"):
            if key not in d:
                raise ConfigError(f"config.json lacks the key {key!r}")
        return cls(width=int(d["width"]), tokens=int(d["tokens"]), longest=int(d.get("longest", 512)))

    def to_dict(self):
        return {"architectures": [self.architecture], "width": self.width, "tokens": self.tokens, "longest": self.longest}


register_architecture(ToyConfig.architecture, ToyConfig, lambda cfg: toy_spec(cfg.width, cfg.tokens))
