"""An architecture that shares nothing with Qwen2's schema is added from this file alone.

Its config.json has none of `hidden_size`, `intermediate_size`, `num_attention_heads`, `head_dim` (it calls its sizes
`d_model`, `n_head`, `d_head`); its layers have one norm and one branch, no feed-forward; its checkpoint uses names of
its own; even layers mix tokens with a running mean kept as fixed-size state, odd layers with the library's attention
under a position encoding that is not a rotate-half table (pairs of neighbours are rotated, by the part's own code).
Everything is registered through the public hooks: an architecture with a configuration class, a block arrangement, a
mixer, a position encoding."""
import math
from dataclasses import dataclass

import pytest
import torch

import helpers
import plain_impl
import mini_llama_cpp_release_b200 as ml
from mini_llama_cpp_release_b200.config import (ConfigError, LayerSpec, ModelConfig, ModelSpec, PartSpec, build_part,
                                                sequential_schedule)
from mini_llama_cpp_release_b200.config.model_config import as_int
from mini_llama_cpp_release_b200.engine import MiniBatch
from mini_llama_cpp_release_b200.parts import Part, StateSpec, TensorSpec

@dataclass(frozen=True, kw_only=True)
class ToyMeanConfig(ModelConfig):
    d_model: int
    n_layer: int
    n_head: int
    d_head: int
    eps: float = 1e-5
    rope_base: float = 100.0

    @classmethod
    def parse(cls, raw):
        own = ("d_model", "n_layer", "n_head", "d_head", "eps", "rope_base")
        cfg = cls(**cls.shared_fields(raw), d_model=as_int(raw, "d_model"), n_layer=as_int(raw, "n_layer"),
                  n_head=as_int(raw, "n_head"), d_head=as_int(raw, "d_head"), eps=float(raw.get("eps", 1e-5)),
                  rope_base=float(raw.get("rope_base", 100.0)),
                  extra={k: v for k, v in raw.items() if k not in cls.SHARED_KEYS and k not in own})
        cfg.validate()
        return cfg

    def validate(self):
        super().validate()
        if self.d_head % 2:
            raise ConfigError("d_head must be even")


def rotate_neighbours(x, positions, base):
    """Pairs (2i, 2i+1) of every head rotated by position · base^(-2i/d): the other customary pairing
    (the reference's RopeType::Normal, src/ops.cpp:170-178 rotates halves instead)."""
    d = x.shape[-1]
    freq = 1.0 / (base ** (torch.arange(0, d, 2, dtype=torch.float32, device=x.device) / d))
    ang = positions.to(torch.float32)[:, None, None] * freq
    c, s = torch.cos(ang), torch.sin(ang)
    a, b = x[..., 0::2], x[..., 1::2]
    return torch.stack([a * c - b * s, a * s + b * c], dim=-1).reshape(x.shape)


@ml.register_part("position", "toy_neighbour_pairs")
class NeighbourPairs(Part):
    graph_safe = True
    fusable = False                     # not a rotate-half table: the attention part calls rotate()

    def __init__(self, name, base):
        super().__init__(name, base=base)
        self.base = base

    def rotate(self, x, positions, out_dtype=None):
        return rotate_neighbours(x.float(), positions, self.base).to(out_dtype or torch.float32)


@ml.register_part("mixer", "toy_running_mean")
class RunningMean(Part):
    """y_t = W_out · mean_{j <= t} (W_in · h_j); the sum so far is the state.  No host round trip."""
    graph_safe = True

    def __init__(self, name, width, inner):
        super().__init__(name, width=width, inner=inner)
        self.width, self.inner = width, inner

    def tensors(self):
        return [TensorSpec(self.name + "in.weight", (self.inner, self.width)),
                TensorSpec(self.name + "out.weight", (self.width, self.inner))]

    def cache_need(self):
        return None

    def state_spec(self):
        return StateSpec((self.inner,), torch.float32)

    def bind(self, get, runtime):
        super().bind(get, runtime)
        self.w_in, self.w_out = get(self.name + "in.weight").float(), get(self.name + "out.weight").float()

    def forward(self, h, step, memory):
        u = h.float() @ self.w_in.t()
        seq = step.tok_seq.long()
        pos = step.positions
        causal = ((seq[:, None] == seq[None, :]) & (pos[:, None] >= pos[None, :])).float()
        sums = causal @ u + memory.state.index_select(0, step.slots_long).index_select(0, seq)
        memory.state.index_copy_(0, step.slots_long, sums.index_select(0, step.cu_seqlens[1:].long() - 1))
        return (sums / (pos.float()[:, None] + 1.0)) @ self.w_out.t()


@ml.register_part("block", "toy_one_branch")
class OneBranch(Part):
    """x ← x + mixer(norm(x)): one norm, one branch."""
    graph_safe = True

    def __init__(self, name, norm, mixer):
        super().__init__(name)
        self.norm = build_part(norm, name + "ln.")
        self.mixer = build_part(mixer, name + "mix.")

    def children(self):
        return (self.norm, self.mixer)

    def forward(self, x, pending, step, memory):
        return x, self.mixer.forward(self.norm.forward(x, pending), step, memory)     # the next norm adds the branch


@ml.register_architecture("ToyMeanLM", config_class=ToyMeanConfig)
def toy_mean_lm(c: ToyMeanConfig) -> ModelSpec:
    norm = PartSpec("norm", "rmsnorm", dict(size=c.d_model, eps=c.eps))
    mean = PartSpec("mixer", "toy_running_mean", dict(width=c.d_model, inner=c.extra["mean_width"]))
    attn = PartSpec("mixer", "gqa_attention", dict(
        hidden_size=c.d_model, num_heads=c.n_head, num_kv_heads=1, head_dim=c.d_head, qkv_bias=True,
        position=PartSpec("position", "toy_neighbour_pairs", dict(base=c.rope_base))))
    layers = tuple(LayerSpec(f"h.{i}.", PartSpec("block", "toy_one_branch", dict(norm=norm, mixer=mean if i % 2 == 0 else attn)))
                   for i in range(c.n_layer))
    return ModelSpec(c, PartSpec("embedding", "token_embedding", dict(vocab_size=c.vocab_size, hidden_size=c.d_model)),
                     layers, sequential_schedule(c.n_layer), norm,
                     PartSpec("head", "linear_head", dict(vocab_size=c.vocab_size, hidden_size=c.d_model)),
                     names={"embedding": "wte.", "final_norm": "ln_f.", "head": "head."})


RAW = dict(architectures=["ToyMeanLM"], vocab_size=150, max_position_embeddings=300, d_model=40, n_layer=4, n_head=2,
           d_head=16, eps=1e-5, rope_base=50.0, mean_width=24)


def plain_logits(folder, tokens):
    w = plain_impl.read_weights(folder)
    T = len(tokens)
    x = plain_impl.embedding(w["wte.weight"], tokens)
    pos = torch.arange(T)
    for i in range(RAW["n_layer"]):
        p = f"h.{i}."
        h = plain_impl.rmsnorm(x, w[p + "ln.weight"], RAW["eps"])
        if i % 2 == 0:
            u = h @ w[p + "mix.in.weight"].t()
            x = x + (torch.cumsum(u, 0) / (pos[:, None] + 1.0)) @ w[p + "mix.out.weight"].t()
        else:
            H, hd = RAW["n_head"], RAW["d_head"]
            q = plain_impl.linear(h, w[p + "mix.q_proj.weight"], w[p + "mix.q_proj.bias"]).view(T, H, hd)
            k = plain_impl.linear(h, w[p + "mix.k_proj.weight"], w[p + "mix.k_proj.bias"]).view(T, 1, hd)
            v = plain_impl.linear(h, w[p + "mix.v_proj.weight"], w[p + "mix.v_proj.bias"]).view(T, 1, hd)
            o = plain_impl.attention(rotate_neighbours(q, pos, RAW["rope_base"]), rotate_neighbours(k, pos, RAW["rope_base"]), v)
            x = x + plain_impl.linear(o.reshape(T, H * hd), w[p + "mix.o_proj.weight"])
    return plain_impl.linear(plain_impl.rmsnorm(x, w["ln_f.weight"], RAW["eps"]), w["head.weight"])


def test_the_shared_configuration_asks_only_for_what_the_engine_reads():
    c = ModelConfig.from_dict(RAW)
    assert isinstance(c, ToyMeanConfig) and (c.d_model, c.n_head, c.extra) == (40, 2, {"mean_width": 24})
    assert ModelConfig.from_dict(c.to_dict()) == c
    for key in ("hidden_size", "intermediate_size", "num_attention_heads", "head_dim"):
        assert key not in c.to_dict()
    with pytest.raises(ConfigError, match="d_model"):
        ModelConfig.from_dict({k: v for k, v in RAW.items() if k != "d_model"})
    with pytest.raises(ConfigError, match="vocab_size"):
        ModelConfig.from_dict({k: v for k, v in RAW.items() if k != "vocab_size"})


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_architecture_builds_loads_steps_and_generates(dtype, tmp_path):
    folder = ml.write_random_model(ModelConfig.from_dict(RAW), str(tmp_path / "toy"), 11, std=0.1)
    llm = ml.load(folder, dtype=dtype, max_tokens=1024, max_seqs=4)
    ctx, cache = llm.context, llm.context.cache
    assert [s is not None for s in cache.state] == [True, False, True, False] and len(cache.groups) == 1
    assert cache.groups[0].entries == [1, 3] and cache.bytes_per_token() == 2 * 2 * 1 * 16 * (4 if dtype == "float32" else 2)
    tol = 2e-5 if dtype == "float32" else 3e-2
    err = lambda got, ref: float((got.double().cpu() - ref.double()).abs().max() / ref.abs().max())
    seqs = [helpers.random_tokens(n, 150, 40 + n) for n in (70, 9, 31)]
    want = [plain_logits(folder, s) for s in seqs]
    # whole, each alone (the 70-token one is a step of a shape that comes again: issued, then warmed up and captured, then replayed)
    for _ in range(3):
        for s, ref in zip(seqs, want):
            slot = ctx.acquire()
            assert err(ctx.forward_batch(MiniBatch.from_tokens(slot, s, want=list(range(len(s))))), ref) <= tol
            ctx.release(slot)
    # unequal prompts together, then one token each; shorter ones end earlier
    heads = [40, 2, 20]
    slots = [ctx.acquire() for _ in seqs]
    out = ctx.forward_batch(MiniBatch.prefill(slots, [s[:h] for s, h in zip(seqs, heads)]))
    for i, h in enumerate(heads):
        assert err(out[i], want[i][h - 1]) <= tol
    live, t = [0, 1, 2], 0
    while live:
        out = ctx.forward_batch(MiniBatch.decode([slots[i] for i in live], [seqs[i][heads[i] + t] for i in live]))
        for row, i in enumerate(live):
            assert err(out[row], want[i][heads[i] + t]) <= tol, (i, t)
        t += 1
        for i in [i for i in live if heads[i] + t == len(seqs[i])]:
            ctx.release(slots[i])
        live = [i for i in live if heads[i] + t < len(seqs[i])]
    cache.check()
    # generation through the entry point: captured decode steps, state advanced once a step
    prompts = [s[:5] for s in seqs]
    seen = []
    gen = llm.generate(prompts, n_predict=12, stop_token_ids=[],
                       on_step=lambda live, chosen, logits: seen.append((list(live), logits.float().cpu().clone())))
    refs = [plain_logits(folder, p + g) for p, g in zip(prompts, gen)]
    for k, (live, logits) in enumerate(seen):
        for row, i in enumerate(live):
            assert err(logits[row], refs[i][4 + k]) <= tol, (k, i)
    assert cache.slots.n_held == 0
