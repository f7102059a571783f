"""Each part of a layer alone against the plain implementation's function for it, and the generality of the
assembly: a toy mixer with state of its own, a layer that runs twice, and a layer that reads another layer's
cache -- all registered from here, without a change to the package's files."""
from dataclasses import dataclass

import numpy as np
import pytest
import torch

import plain_qwen3 as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def build_ctx(dtype):
    from vllm_cpp_b200.parts import BuildContext
    return BuildContext(dtype, torch.device(DEV))


def store_of(tensors, dtype):
    from vllm_cpp_b200.weights import WeightStore
    return WeightStore(tensors, dtype, DEV)


def tol(dtype):
    return dict(rtol=1e-4, atol=1e-5) if dtype == torch.float32 else dict(rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_part(dtype):
    from vllm_cpp_b200.parts import RMSNorm
    H, T, eps = 96, 5, 1e-5
    w = (1 + 0.1 * torch.randn(H)).to(torch.bfloat16)
    part = RMSNorm({"size": H, "eps": eps}, "n.", build_ctx(dtype))
    assert [s.name for s in part.tensor_specs()] == ["n.weight"]
    part.bind(store_of({"n.weight": w}, dtype))
    resid, delta = torch.randn(T, H, device=DEV), torch.randn(2, T, H, device=DEV)
    want_x = resid.double().cpu() + delta.double().cpu().sum(0)
    y = part.forward(resid, delta)
    torch.testing.assert_close(y.double().cpu(), P.rms_norm(want_x, w.double(), eps), **tol(dtype))
    torch.testing.assert_close(resid.double().cpu(), want_x, rtol=1e-6, atol=1e-6)     # the stream took the deltas


def test_rotary_table():
    from vllm_cpp_b200.parts import RotaryEmbedding
    part = RotaryEmbedding({"head_dim": 32, "theta": 1e6, "max_positions": 300}, "", build_ctx(torch.float32))
    cos, sin = P.rope_angles(32, 1e6, list(range(300)))
    torch.testing.assert_close(part.table.cpu().double(), torch.cat([cos, sin], 1), rtol=0, atol=1e-7)
    other = RotaryEmbedding({"head_dim": 32, "theta": 1e6, "max_positions": 300}, "x.", part.build)
    assert other.table is part.table                                                  # equal parameters share one table


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T", [3, 150])
def test_swiglu_part(dtype, T):
    from vllm_cpp_b200.parts import SwiGLUMLP
    H, I = 96, 200
    w = {f"m.{n}_proj.weight": (0.1 * torch.randn(*s)).to(torch.bfloat16)
         for n, s in (("gate", (I, H)), ("up", (I, H)), ("down", (H, I)))}
    part = SwiGLUMLP({"hidden_size": H, "intermediate_size": I}, "m.", build_ctx(dtype))
    part.bind(store_of(w, dtype))
    x = torch.randn(T, H).to(torch.bfloat16)

    class Ctx:
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
    y = part.forward(x.to(DEV).to(dtype), Ctx())
    y = y.double().cpu().sum(0) if y.dim() == 3 else y.double().cpu()
    want = P.swiglu_mlp(x.double(), *(w[f"m.{n}_proj.weight"].double() for n in ("gate", "up", "down")))
    torch.testing.assert_close(y, want, **tol(dtype))
    assert Ctx.status.item() == 0


class OnePartModel:
    """Just enough of a model for ModelRunner: one mixer, one cache, returns the mixer's output rows."""

    def __init__(self, mixer, hidden, x_by_token):
        self.mixer, self.x = mixer, x_by_token

        class Spec:
            vocab_size, max_positions = x_by_token.shape[0], 4096
        self.spec = Spec()

    def cache_specs(self):
        return {0: self.mixer.cache_spec()}

    def forward(self, ctx, caches):
        x = self.x[ctx.token_ids.long()]                # "embedding": token id t stands for row t of x
        d = self.mixer.forward(x, ctx, caches[0], True)
        return d.sum(0) if d.dim() == 3 else d


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,window", [(4, 2, 16, 0), (6, 2, 32, 9), (8, 2, 64, 0), (4, 4, 128, 40)])
def test_attention_part_in_portions(dtype, nh, nkv, hd, window):
    """The attention mixer alone, fed one sequence in portions (17, 1, 1, 30, 2, ...) through the paged cache."""
    from vllm_cpp_b200.engine.step import ModelRunner, StepEntry
    from vllm_cpp_b200.parts import GQAAttention
    from vllm_cpp_b200.registry import PartSpec
    from vllm_cpp_b200.runtime import runtime
    H, T, eps, theta, ps = 72, 90, 1e-6, 1e4, 8
    torch.manual_seed(nh * hd)
    w = {"a.q_proj.weight": 0.15 * torch.randn(nh * hd, H), "a.k_proj.weight": 0.15 * torch.randn(nkv * hd, H),
         "a.v_proj.weight": 0.15 * torch.randn(nkv * hd, H), "a.o_proj.weight": 0.15 * torch.randn(H, nh * hd),
         "a.q_norm.weight": 1 + 0.1 * torch.randn(hd), "a.k_norm.weight": 1 + 0.1 * torch.randn(hd)}
    w = {k: v.to(torch.bfloat16) for k, v in w.items()}
    rope = PartSpec("rope", {"head_dim": hd, "theta": theta, "max_positions": 4096})
    part = GQAAttention({"hidden_size": H, "num_heads": nh, "num_kv_heads": nkv, "head_dim": hd, "eps": eps,
                         "qk_norm": True, "window": window, "position": rope}, "a.", build_ctx(dtype))
    part.bind(store_of(w, dtype))
    x = torch.randn(T, H).to(torch.bfloat16)
    runner = ModelRunner(OnePartModel(part, H, x.to(DEV).to(dtype)), ps, 32, 2, dtype, DEV, cuda_graphs=False)
    rt = runtime()
    cm = rt.CacheManager(runner.layout.runtime_groups(rt, ps, 32), 2)
    cm.open(0)
    got, p = [], 0
    for n in [17, 1, 1, 30, 2, 1, 38]:
        assert cm.reserve(0, p + n)
        out = runner.step([StepEntry(cm.slot(0), p, list(range(p, p + n)), [cm.block_table(0, 0)], list(range(n)))])
        cm.commit(0, p + n)
        got.append(out.double().cpu())
        p += n
    got = torch.cat(got)
    # the same in the plain implementation's functions
    W = {k: v.double() for k, v in w.items()}
    xd = x.double()
    q = P.head_rms_norm(P.linear(xd, W["a.q_proj.weight"]).view(T, nh, hd), W["a.q_norm.weight"], eps)
    k = P.head_rms_norm(P.linear(xd, W["a.k_proj.weight"]).view(T, nkv, hd), W["a.k_norm.weight"], eps)
    v = P.linear(xd, W["a.v_proj.weight"]).view(T, nkv, hd)
    cos, sin = P.rope_angles(hd, theta, list(range(T)))
    a = P.attention(P.rope_half_split(q, cos, sin), P.rope_half_split(k, cos, sin), v, window or None)
    want = P.linear(a.reshape(T, nh * hd), W["a.o_proj.weight"])
    torch.testing.assert_close(got, want, **tol(dtype))
    if window:
        assert cm.block_table(0, 0)[0] == -1         # pages the window has passed were given back on the way


# ----------------------------------------------------------------------------------------------------------
# a toy architecture, defined here: a mixer with state of its own, a layer run twice, a layer reading another's cache
# ----------------------------------------------------------------------------------------------------------

@dataclass(frozen=True)
class ToyConfig:
    vocab_size: int = 97
    hidden_size: int = 48
    intermediate_size: int = 80
    num_heads: int = 4
    num_kv_heads: int = 2
    head_dim: int = 16
    eps: float = 1e-5
    theta: float = 1e4
    max_positions: int = 128
    architecture: str = "ToyForCausalLM"

    @classmethod
    def from_dict(cls, d):
        return cls(**{k: d[k] for k in cls.__dataclass_fields__ if k in d and k != "architecture"})

    def to_dict(self):
        d = {k: getattr(self, k) for k in self.__dataclass_fields__ if k != "architecture"}
        d["architectures"] = [self.architecture]
        return d


PRIOR = 0.25      # what the running-mean mixer's state holds before a request's first token


def register_toy():
    from vllm_cpp_b200.parts import CacheSpec, Mixer
    from vllm_cpp_b200.registry import LayerRun, LayerSpec, ModelSpec, PartSpec, register_architecture, register_part
    from vllm_cpp_b200.weights import TensorSpec

    class RunningMeanMixer(Mixer):
        """delta_t = W . mean(PRIOR, x_0..x_t): needs the running sum of a request's inputs, a state of fixed size
        that starts at PRIOR in every lane (the cache sets it when a request's first tokens arrive)."""
        capturable = False

        def cache_spec(self):
            return CacheSpec("state", shape=(int(self.params["size"]),), dtype="float32", initial_value=PRIOR)

        def tensor_specs(self):
            n = int(self.params["size"])
            return [TensorSpec(self.prefix + "mix.weight", (n, n))]

        def bind(self, store):
            self.w = store.matrix(self.prefix + "mix.weight")

        def forward(self, x, ctx, cache, writes=True):
            out = torch.empty(x.shape, dtype=torch.float32, device=x.device)
            for i, e in enumerate(ctx.entries):
                s, n = ctx.host_q_start[i], len(e.tokens)
                run = cache.state[e.slot] + torch.cumsum(x[s:s + n].float(), 0)
                cache.state[e.slot] = run[-1]
                count = torch.arange(e.start_pos + 2, e.start_pos + n + 2, device=x.device, dtype=torch.float32)
                out[s:s + n] = run / count[:, None]
            return out @ self.w.float().T

    def describe(cfg: ToyConfig):
        H = cfg.hidden_size
        norm = PartSpec("rmsnorm", {"size": H, "eps": cfg.eps})
        ffn = PartSpec("swiglu", {"hidden_size": H, "intermediate_size": cfg.intermediate_size})
        rope = PartSpec("rope", {"head_dim": cfg.head_dim, "theta": cfg.theta, "max_positions": cfg.max_positions})
        attn = dict(hidden_size=H, num_heads=cfg.num_heads, num_kv_heads=cfg.num_kv_heads, head_dim=cfg.head_dim,
                    eps=cfg.eps, qk_norm=True, window=0, position=rope)

        def layer(i, mixer):
            return LayerSpec(prefix=f"toy.{i}.", block=PartSpec("prenorm"),
                             parts={"norm1": (norm, "n1."), "mixer": (mixer, "mix."), "norm2": (norm, "n2."),
                                    "feed_forward": (ffn, "ff.")})
        layers = (layer(0, PartSpec("gqa_attention", dict(attn, has_kv=True))),
                  layer(1, PartSpec("running_mean", {"size": H})),
                  layer(2, PartSpec("gqa_attention", dict(attn, has_kv=False))))
        order = (LayerRun(0, 0), LayerRun(1, 1), LayerRun(0, 2), LayerRun(2, 0, writes=False), LayerRun(1, 3))
        return ModelSpec(hidden_size=H, vocab_size=cfg.vocab_size, max_positions=cfg.max_positions,
                         embed_tensor="toy.embed.weight", layers=layers, order=order, final_norm=norm,
                         final_norm_prefix="toy.norm.", lm_head_tensor=None)

    register_part("mixer", "running_mean", RunningMeanMixer)
    register_architecture("ToyForCausalLM", ToyConfig, describe)


def plain_toy(cfg: ToyConfig, W, ids):
    """The toy model on one whole sequence, from the plain implementation's functions."""
    T, nh, nkv, hd = len(ids), cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
    cos, sin = P.rope_angles(hd, cfg.theta, list(range(T)))
    x = P.embed(ids, W["toy.embed.weight"])
    kept = {}

    def attn_layer(i, x, own_kv, key):
        p = f"toy.{i}."
        y = P.rms_norm(x, W[p + "n1.weight"], cfg.eps)
        q = P.rope_half_split(P.head_rms_norm(P.linear(y, W[p + "mix.q_proj.weight"]).view(T, nh, hd), W[p + "mix.q_norm.weight"], cfg.eps), cos, sin)
        if own_kv:
            k = P.rope_half_split(P.head_rms_norm(P.linear(y, W[p + "mix.k_proj.weight"]).view(T, nkv, hd), W[p + "mix.k_norm.weight"], cfg.eps), cos, sin)
            kept[key] = (k, P.linear(y, W[p + "mix.v_proj.weight"]).view(T, nkv, hd))
        k, v = kept[key]
        x = x + P.linear(P.attention(q, k, v).reshape(T, nh * hd), W[p + "mix.o_proj.weight"])
        y = P.rms_norm(x, W[p + "n2.weight"], cfg.eps)
        return x + P.swiglu_mlp(y, W[p + "ff.gate_proj.weight"], W[p + "ff.up_proj.weight"], W[p + "ff.down_proj.weight"])

    def mean_layer(x):
        p = "toy.1."
        y = P.rms_norm(x, W[p + "n1.weight"], cfg.eps)
        mean = (PRIOR + torch.cumsum(y, 0)) / torch.arange(2, T + 2, dtype=torch.float64)[:, None]
        x = x + P.linear(mean, W[p + "mix.mix.weight"])
        y = P.rms_norm(x, W[p + "n2.weight"], cfg.eps)
        return x + P.swiglu_mlp(y, W[p + "ff.gate_proj.weight"], W[p + "ff.up_proj.weight"], W[p + "ff.down_proj.weight"])

    x = attn_layer(0, x, True, 0)
    x = mean_layer(x)
    x = attn_layer(0, x, True, 2)       # the same layer again, with a cache of its own
    x = attn_layer(2, x, False, 0)      # queries of layer 2 over the keys the first run of layer 0 stored
    x = mean_layer(x)                   # and the stateful layer again, with a second state
    return P.linear(P.rms_norm(x, W["toy.norm.weight"], cfg.eps), W["toy.embed.weight"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_architecture_registers_builds_and_steps(dtype, tmp_path):
    from vllm_cpp_b200 import load_config, write_random_model, unregister_architecture, unregister_part
    from vllm_cpp_b200.engine.llm import TORCH_DTYPES
    from vllm_cpp_b200.engine.step import ModelRunner, StepEntry
    from vllm_cpp_b200.models import build_model
    from vllm_cpp_b200.runtime import runtime
    from vllm_cpp_b200.weights import open_model_weights
    register_toy()
    try:
        cfg = ToyConfig()
        folder = write_random_model(cfg, 3, tmp_path / "toy")
        assert load_config(folder) == cfg
        _, W = P.read_model(folder)
        W = {k: v.double() for k, v in W.items()}
        assert "toy.2.mix.k_proj.weight" not in W and "toy.1.mix.mix.weight" in W     # the reader of a cache has no K/V weights
        td = TORCH_DTYPES[dtype]
        model = build_model(cfg, td, DEV)
        store = open_model_weights(folder, td, DEV)
        model.load(store)
        assert not model.capturable
        ps = 4
        runner = ModelRunner(model, ps, 64, 3, td, DEV)
        kinds = [(g.spec.kind, len(g.cache_ids)) for g in runner.layout.groups]
        assert kinds == [("kv", 2), ("state", 2)]          # caches 0 and 2 share pages; 1 and 3 are two states per slot
        rt = runtime()
        cm = rt.CacheManager(runner.layout.runtime_groups(rt, ps, 64), 3)
        rng = np.random.default_rng(0)
        seqs = {r: rng.integers(0, cfg.vocab_size, n).tolist() for r, n in ((0, 50), (1, 23), (2, 9))}
        want = {r: plain_toy(cfg, W, t) for r, t in seqs.items()}
        pos = {r: 0 for r in seqs}
        cuts = {0: [7, 1, 20, 2, 1, 19], 1: [1, 1, 21], 2: [9]}
        for r in seqs:
            cm.open(r)
        worst = 0.0
        for step in range(6):
            entries, rows = [], []
            for r in seqs:
                if step < len(cuts[r]):
                    n = cuts[r][step]
                    assert cm.reserve(r, pos[r] + n)
                    entries.append(StepEntry(cm.slot(r), pos[r], seqs[r][pos[r]:pos[r] + n], [cm.block_table(r, 0)], list(range(n))))
                    rows += [(r, pos[r] + i) for i in range(n)]
                    pos[r] += n
            out = runner.step(entries).double().cpu()
            for r in seqs:
                cm.commit(r, pos[r])
            ref = torch.stack([want[r][p] for r, p in rows])
            worst = max(worst, ((out - ref).abs().max() / ref.abs().max()).item())
        assert worst < (2e-5 if dtype == "float32" else 4e-2), worst
        # a slot handed to another request starts from a clean state
        cm.close(2)
        cm.open(7)
        assert cm.slot(7) == 2 and cm.reserve(7, 9)
        out = runner.step([StepEntry(2, 0, seqs[2], [cm.block_table(7, 0)], [8])]).double().cpu()
        assert ((out[0] - want[2][8]).abs().max() / want[2][8].abs().max()).item() < (2e-5 if dtype == "float32" else 4e-2)
    finally:
        unregister_architecture("ToyForCausalLM")
        unregister_part("mixer", "running_mean")


# ----------------------------------------------------------------------------------------------------------
# a second toy architecture: a feed-forward with routing and another position encoding, both defined here
# ----------------------------------------------------------------------------------------------------------

@dataclass(frozen=True)
class RoutedToyConfig:
    vocab_size: int = 61
    hidden_size: int = 40
    expert_size: int = 24
    num_experts: int = 3
    num_heads: int = 5
    num_kv_heads: int = 1
    head_dim: int = 16
    eps: float = 1e-6
    theta: float = 500.0
    position_scale: float = 4.0
    rotary_dim: int = 8            # of the 16 lanes of a head, paired (2i, 2i+1)
    embedding_scale: float = 3.0
    logit_cap: float = 2.0
    second_layer_page_size: int = 16
    max_positions: int = 96
    num_layers: int = 2
    architecture: str = "RoutedToyForCausalLM"

    @classmethod
    def from_dict(cls, d):
        return cls(**{k: d[k] for k in cls.__dataclass_fields__ if k in d and k != "architecture"})

    def to_dict(self):
        d = {k: getattr(self, k) for k in self.__dataclass_fields__ if k != "architecture"}
        d["architectures"] = [self.architecture]
        return d


def register_routed_toy():
    from vllm_cpp_b200.parts import GQAAttention, LMHead, TokenEmbedding
    from vllm_cpp_b200.parts.base import FeedForward, PositionEncoding
    from vllm_cpp_b200.registry import LayerRun, LayerSpec, ModelSpec, PartSpec, register_architecture, register_part
    from vllm_cpp_b200.weights import TensorSpec

    class TopOneExperts(FeedForward):
        """Router logits in 32-bit, the best expert per token (lowest index wins ties), its SwiGLU scaled by the
        router's softmax weight.  Plain tensor code: a toy for the interfaces, not a kernel."""

        def tensor_specs(self):
            H, I, E, p = int(self.params["hidden_size"]), int(self.params["expert_size"]), int(self.params["num_experts"]), self.prefix
            specs = [TensorSpec(p + "router.weight", (E, H))]
            for e in range(E):
                specs += [TensorSpec(f"{p}experts.{e}.gate.weight", (I, H)), TensorSpec(f"{p}experts.{e}.up.weight", (I, H)),
                          TensorSpec(f"{p}experts.{e}.down.weight", (H, I))]
            return specs

        def bind(self, store):
            E, p = int(self.params["num_experts"]), self.prefix
            self.router = store.matrix(p + "router.weight")
            self.experts = [tuple(store.matrix(f"{p}experts.{e}.{n}.weight") for n in ("gate", "up", "down")) for e in range(E)]

        def forward(self, x, ctx):
            logits = x.float() @ self.router.float().T
            prob = torch.softmax(logits, -1)
            best = torch.argmax(logits, -1)
            out = torch.zeros(x.shape, dtype=torch.float32, device=x.device)
            for e, (g, u, d) in enumerate(self.experts):
                xe = x.float()
                h = torch.nn.functional.silu(xe @ g.float().T) * (xe @ u.float().T)
                out += torch.where((best == e)[:, None], prob[:, e:e + 1] * (h.to(x.dtype).float() @ d.float().T), 0.0)
            return out

    class ScaledRotary(PositionEncoding):
        """Rotary angles of position / scale on the first ``rotary_dim`` lanes of a head, paired (2i, 2i+1): what the
        attention part asks of its position part is ``table``, ``rotary_dim`` and ``pairing``."""

        def __init__(self, params, prefix, build):
            super().__init__(params, prefix, build)
            rd, theta, scale, n = int(params["rotary_dim"]), float(params["theta"]), float(params["scale"]), int(params["max_positions"])
            inv = theta ** (-2.0 * torch.arange(rd // 2, dtype=torch.float64) / rd)
            ang = (torch.arange(n, dtype=torch.float64) / scale)[:, None] * inv[None, :]
            self.table = torch.cat([torch.cos(ang), torch.sin(ang)], 1).float().contiguous().to(build.device)
            self.rotary_dim, self.pairing = rd, "interleaved"

    class ScaledEmbedding(TokenEmbedding):
        """x = scale * E[id]: an embedding of another kind, registered from here."""

        def forward(self, ids, n_tokens, status):
            return super().forward(ids, n_tokens, status) * float(self.params["scale"])

    class CappedHead(LMHead):
        """logits = cap * tanh(logits / cap): a head of another kind."""

        def forward(self, y, status=None):
            cap = float(self.params["cap"])
            return cap * torch.tanh(super().forward(y, status) / cap)

    class PagedAttention(GQAAttention):
        """The package's attention with pages of a size of its own: its caches get a pool of their own."""

        def cache_spec(self):
            import dataclasses
            return dataclasses.replace(super().cache_spec(), page_size=int(self.params["page_size"]))

    def describe(cfg: RoutedToyConfig):
        H = cfg.hidden_size
        norm = PartSpec("rmsnorm", {"size": H, "eps": cfg.eps})
        ffn = PartSpec("top_one_experts", {"hidden_size": H, "expert_size": cfg.expert_size, "num_experts": cfg.num_experts})
        pos = PartSpec("scaled_rotary", {"rotary_dim": cfg.rotary_dim, "theta": cfg.theta, "scale": cfg.position_scale,
                                         "max_positions": cfg.max_positions})
        attn = dict(hidden_size=H, num_heads=cfg.num_heads, num_kv_heads=cfg.num_kv_heads, head_dim=cfg.head_dim,
                    eps=cfg.eps, qk_norm=True, window=0, position=pos)
        # the first layer's keys lie in pages of the engine's size, the second layer's in pages of its own
        mixers = [PartSpec("gqa_attention", attn)] + [PartSpec("paged_attention", dict(attn, page_size=cfg.second_layer_page_size))] * (cfg.num_layers - 1)
        # the roles of a layer may name their families themselves (here as the defaults would)
        layers = tuple(LayerSpec(prefix=f"rt.{i}.", block=PartSpec("prenorm"),
                                 parts={"norm1": (norm, "n1.", "norm"), "mixer": (mixers[i], "att.", "mixer"), "norm2": (norm, "n2."),
                                        "feed_forward": (ffn, "moe.")}) for i in range(cfg.num_layers))
        return ModelSpec(hidden_size=H, vocab_size=cfg.vocab_size, max_positions=cfg.max_positions,
                         embed_tensor=None, layers=layers,
                         order=tuple(LayerRun(i, i) for i in range(cfg.num_layers)), final_norm=norm,
                         final_norm_prefix="rt.norm.", lm_head_tensor=None,
                         embedding=PartSpec("scaled_embedding", {"tensor": "rt.embed.weight", "vocab_size": cfg.vocab_size,
                                                                 "hidden_size": H, "scale": cfg.embedding_scale}),
                         head=PartSpec("capped_head", {"tensor": "rt.head.weight", "vocab_size": cfg.vocab_size,
                                                       "hidden_size": H, "cap": cfg.logit_cap}))

    register_part("feed_forward", "top_one_experts", TopOneExperts)
    register_part("position", "scaled_rotary", ScaledRotary)
    register_part("embedding", "scaled_embedding", ScaledEmbedding)
    register_part("head", "capped_head", CappedHead)
    register_part("mixer", "paged_attention", PagedAttention)
    register_architecture("RoutedToyForCausalLM", RoutedToyConfig, describe)


def plain_routed_toy(cfg: RoutedToyConfig, W, ids, act_dtype):
    T, nh, nkv, hd = len(ids), cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
    rd = cfg.rotary_dim
    inv = cfg.theta ** (-2.0 * torch.arange(rd // 2, dtype=torch.float64) / rd)
    ang = (torch.arange(T, dtype=torch.float64) / cfg.position_scale)[:, None] * inv[None, :]
    cos, sin = torch.cos(ang).float().double(), torch.sin(ang).float().double()

    def rotate(h):      # the first rd lanes of every head turn, paired (2i, 2i+1); the rest pass
        return torch.cat([P.rope_interleaved(h[..., :rd], cos, sin), h[..., rd:]], -1)

    x = cfg.embedding_scale * P.embed(ids, W["rt.embed.weight"])
    for i in range(cfg.num_layers):
        p = f"rt.{i}."
        y = P.rms_norm(x, W[p + "n1.weight"], cfg.eps)
        q = rotate(P.head_rms_norm(P.linear(y, W[p + "att.q_proj.weight"]).view(T, nh, hd), W[p + "att.q_norm.weight"], cfg.eps))
        k = rotate(P.head_rms_norm(P.linear(y, W[p + "att.k_proj.weight"]).view(T, nkv, hd), W[p + "att.k_norm.weight"], cfg.eps))
        v = P.linear(y, W[p + "att.v_proj.weight"]).view(T, nkv, hd)
        x = x + P.linear(P.attention(q, k, v).reshape(T, nh * hd), W[p + "att.o_proj.weight"])
        y = P.rms_norm(x, W[p + "n2.weight"], cfg.eps)
        logits = P.linear(y, W[p + "moe.router.weight"])
        prob, best = torch.softmax(logits, -1), torch.argmax(logits, -1)
        d = torch.zeros_like(x)
        for t in range(T):
            e = int(best[t])
            h = P.linear(y[t:t + 1], W[f"{p}moe.experts.{e}.gate.weight"])
            h = h / (1 + torch.exp(-h)) * P.linear(y[t:t + 1], W[f"{p}moe.experts.{e}.up.weight"])
            d[t] = prob[t, e] * P.linear(h, W[f"{p}moe.experts.{e}.down.weight"])[0]
        x = x + d
    logits = P.linear(P.rms_norm(x, W["rt.norm.weight"], cfg.eps), W["rt.head.weight"])
    return cfg.logit_cap * torch.tanh(logits / cfg.logit_cap), best


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_routed_feed_forward_and_other_positions(dtype, tmp_path):
    """A feed-forward with routing, a position encoding of another kind (scaled positions, half of each head's lanes
    rotated, in interleaved pairs), a scaled embedding, a head that caps its logits, and a second layer whose keys
    lie in pages of another size than the first layer's (two pools, two block tables a request) -- all registered
    from here and run through the unchanged loader, cache, step function and scheduler: portions and batching give
    the plain model's logits, and greedy generation through the entry point gives its tokens."""
    from vllm_cpp_b200 import LLM, EngineConfig, load_config, write_random_model, unregister_architecture, unregister_part
    from vllm_cpp_b200.engine.llm import TORCH_DTYPES
    from vllm_cpp_b200.engine.step import ModelRunner, StepEntry
    from vllm_cpp_b200.models import build_model
    from vllm_cpp_b200.runtime import runtime
    from vllm_cpp_b200.weights import open_model_weights
    register_routed_toy()
    try:
        cfg = RoutedToyConfig()
        folder = write_random_model(cfg, 11, tmp_path / "routed")
        assert load_config(folder) == cfg
        _, W = P.read_model(folder)
        W = {k: v.double() for k, v in W.items()}
        td = TORCH_DTYPES[dtype]
        model = build_model(cfg, td, DEV)
        model.load(open_model_weights(folder, td, DEV))
        ps = 8
        runner = ModelRunner(model, ps, 16, 2, td, DEV)
        assert runner.page_sizes == [ps, cfg.second_layer_page_size] and [t.shape[1] for t in runner.tables] == [12, 6]
        rt = runtime()
        cm = rt.CacheManager(runner.layout.runtime_groups(rt, ps, 16), 2)
        assert cm.num_groups() == 2
        rng = np.random.default_rng(5)
        seqs = {0: rng.integers(0, cfg.vocab_size, 37).tolist(), 1: rng.integers(0, cfg.vocab_size, 12).tolist()}
        want = {r: plain_routed_toy(cfg, W, t, td)[0] for r, t in seqs.items()}
        cuts, pos = {0: [5, 30, 1, 1], 1: [2, 1, 9]}, {0: 0, 1: 0}
        for r in seqs:
            cm.open(r)
        worst = 0.0
        for step in range(4):
            entries, rows = [], []
            for r in seqs:
                if step < len(cuts[r]):
                    n = cuts[r][step]
                    assert cm.reserve(r, pos[r] + n)
                    entries.append(StepEntry(cm.slot(r), pos[r], seqs[r][pos[r]:pos[r] + n],
                                             [cm.block_table(r, g) for g in range(2)], list(range(n))))
                    rows += [(r, pos[r] + i) for i in range(n)]
                    pos[r] += n
            out = runner.step(entries).double().cpu()
            for r in seqs:
                cm.commit(r, pos[r])
            ref = torch.stack([want[r][p] for r, p in rows])
            worst = max(worst, ((out - ref).abs().max() / ref.abs().max()).item())
        # (with this seed no token sits between two experts closely enough for bfloat16 to route it differently)
        assert worst < (2e-5 if dtype == "float32" else 4e-2), worst
        if dtype == "float32":
            llm = LLM(folder, engine=EngineConfig(dtype=dtype, page_size=ps, max_tokens=128, max_num_seqs=2, max_step_tokens=8))
            got = llm.generate([seqs[1]], 6, 0.0, 1.0, repeat_penalty=1.0)[0]
            ids = list(seqs[1])
            for _ in range(6):
                ids.append(int(plain_routed_toy(cfg, W, ids, td)[0][-1].argmax()))
            assert got == ids[len(seqs[1]):]
    finally:
        unregister_architecture("RoutedToyForCausalLM")
        unregister_part("feed_forward", "top_one_experts")
        unregister_part("position", "scaled_rotary")
        unregister_part("embedding", "scaled_embedding")
        unregister_part("head", "capped_head")
        unregister_part("mixer", "paged_attention")
