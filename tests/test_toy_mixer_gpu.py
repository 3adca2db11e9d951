"""A mixer with state of its own, defined here, is registered, built, given random weights,
loaded and stepped through the library's public hooks alone.

The toy mixer keeps one vector per sequence: s ← decay·s + W_in·h_t, y_t = W_out·s.  The toy
architecture alternates it with attention layers, so one model has different mixers in
different layers, a cache group for some runs and fixed-size state for others."""
import pytest
import torch

import helpers
import plain_impl
import mini_llama_cpp_release_b200 as ml
from mini_llama_cpp_release_b200.config import ModelConfig, ModelSpec, PartSpec, prenorm_layer, sequential_schedule
from mini_llama_cpp_release_b200.engine import MiniBatch
from mini_llama_cpp_release_b200.models.qwen2 import LAYER_NAMES
from mini_llama_cpp_release_b200.parts import Part, StateSpec, TensorSpec

pytestmark = pytest.mark.gpu


@ml.register_part("mixer", "toy_decay")
class ToyDecayMixer(Part):
    def __init__(self, name, hidden_size, state_size, decay):
        super().__init__(name, hidden_size=hidden_size, state_size=state_size, decay=decay)
        self.hidden, self.n, self.decay = hidden_size, state_size, decay

    def tensors(self):
        return [TensorSpec(self.name + "in_proj.weight", (self.n, self.hidden)),
                TensorSpec(self.name + "out_proj.weight", (self.hidden, self.n))]

    def cache_need(self):
        return None

    def state_spec(self):
        return StateSpec((self.n,), torch.float32)

    def bind(self, get, runtime):
        super().bind(get, runtime)
        self.w_in = get(self.name + "in_proj.weight").float()
        self.w_out = get(self.name + "out_proj.weight").float()

    def forward(self, h, step, memory):
        u = h.float() @ self.w_in.t()
        y = torch.empty(h.shape[0], self.hidden, dtype=torch.float32, device=h.device)
        cu, slots = step.cu_seqlens.tolist(), step.slots.tolist()
        for b, slot in enumerate(slots):
            s = memory.state[slot]
            for t in range(cu[b], cu[b + 1]):
                s = self.decay * s + u[t]
                y[t] = self.w_out @ s
            memory.state[slot] = s
        return y


@ml.register_part("mixer", "toy_decay_on_device")
class ToyDecayMixerOnDevice(ToyDecayMixer):
    """The same recurrence without a host round trip, so that steps through it may be captured into CUDA graphs:
    s_t = decay^(t - first + 1)·s_before + sum_{j <= t, same sequence} decay^(t - j)·u_j, with every index taken from
    the step's device tensors."""
    graph_safe = True

    def forward(self, h, step, memory):
        u = h.float() @ self.w_in.t()
        seq = step.tok_seq.long()
        pos = step.positions.float()
        same = seq[:, None] == seq[None, :]
        ahead = pos[:, None] - pos[None, :]
        mix = torch.pow(self.decay, ahead.clamp_min(0)) * (same & (ahead >= 0)).float()
        before = memory.state.index_select(0, step.slots_long)                      # [n_seqs, n]
        since = pos - step.start_pos.float().index_select(0, seq) + 1
        s_all = mix @ u + torch.pow(self.decay, since)[:, None] * before.index_select(0, seq)
        last = step.cu_seqlens[1:].long() - 1
        memory.state.index_copy_(0, step.slots_long, s_all.index_select(0, last))
        return s_all @ self.w_out.t()


@ml.register_architecture("ToyDecayLM")
def toy_decay_lm(c: ModelConfig) -> ModelSpec:
    norm = PartSpec("norm", "rmsnorm", dict(size=c.hidden_size, eps=c.rms_norm_eps))
    rope = PartSpec("position", "rope_neox", dict(head_dim=c.head_dim, theta=c.rope_theta, max_positions=c.max_position_embeddings))
    attn = PartSpec("mixer", "gqa_attention", dict(hidden_size=c.hidden_size, num_heads=c.num_attention_heads,
                                                   num_kv_heads=c.num_key_value_heads, head_dim=c.head_dim, qkv_bias=False, position=rope))
    toy = PartSpec("mixer", c.extra.get("toy_kind", "toy_decay"), dict(hidden_size=c.hidden_size, state_size=c.extra["toy_state_size"], decay=c.extra["toy_decay"]))
    ffn = PartSpec("feed_forward", "swiglu", dict(hidden_size=c.hidden_size, intermediate_size=c.intermediate_size))
    layers = tuple(prenorm_layer(f"model.layers.{i}.", toy if i % 2 == 0 else attn, ffn, norm, norm, LAYER_NAMES)
                   for i in range(c.num_hidden_layers))
    return ModelSpec(c, PartSpec("embedding", "token_embedding", dict(vocab_size=c.vocab_size, hidden_size=c.hidden_size)),
                     layers, sequential_schedule(len(layers)), norm,
                     PartSpec("head", "linear_head", dict(vocab_size=c.vocab_size, hidden_size=c.hidden_size)))


RAW = dict(architectures=["ToyDecayLM"], hidden_size=48, intermediate_size=80, num_hidden_layers=3, num_attention_heads=3,
           num_key_value_heads=1, head_dim=16, vocab_size=200, max_position_embeddings=256, rope_theta=1e4,
           rms_norm_eps=1e-5, toy_state_size=20, toy_decay=0.9)


def plain_logits(folder, tokens):
    cfg, w = plain_impl.read_config(folder), plain_impl.read_weights(folder)
    x = plain_impl.embedding(w["model.embed_tokens.weight"], tokens)
    pos = torch.arange(len(tokens))
    for i in range(3):
        p = f"model.layers.{i}."
        h = plain_impl.rmsnorm(x, w[p + "input_layernorm.weight"], 1e-5)
        if i % 2 == 0:
            u = h @ w[p + "self_attn.in_proj.weight"].t()
            s, ys = torch.zeros(20), []
            for t in range(len(tokens)):
                s = 0.9 * s + u[t]
                ys.append(w[p + "self_attn.out_proj.weight"] @ s)
            x = x + torch.stack(ys)
        else:
            x = x + plain_impl.attention_block(h, w, p, cfg, pos, None)
        h2 = plain_impl.rmsnorm(x, w[p + "post_attention_layernorm.weight"], 1e-5)
        x = x + plain_impl.swiglu_ffn(h2, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    return plain_impl.linear(plain_impl.rmsnorm(x, w["model.norm.weight"], 1e-5), w["lm_head.weight"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_mixer_with_state_registers_builds_and_steps(dtype, tmp_path):
    folder = ml.write_random_model(ModelConfig.from_dict(RAW), str(tmp_path / "toy"), 7, std=0.1)
    llm = ml.load(folder, dtype=dtype, max_tokens=1024, max_seqs=4)
    cache = llm.context.cache
    assert [s is not None for s in cache.state] == [True, False, True] and cache.state[0].shape == (4, 20)
    assert len(cache.groups) == 1 and cache.groups[0].entries == [1]
    ctx = llm.context
    seqs = [helpers.random_tokens(n, 200, n) for n in (30, 7, 12)]
    want = [plain_logits(folder, s) for s in seqs]
    tol = 2e-5 if dtype == "float32" else 3e-2

    def err(got, ref):
        return float((got.double().cpu() - ref.double()).abs().max() / ref.abs().max())

    # whole, each alone
    for s, ref in zip(seqs, want):
        slot = ctx.acquire()
        assert err(ctx.forward_batch(MiniBatch.from_tokens(slot, s, want=list(range(len(s))))), ref) <= tol
        ctx.release(slot)
    # together: prompts of unequal length, then one token each; the slots were used before, so state must start at zero
    slots = [ctx.acquire() for _ in seqs]
    heads = [5, 1, 11]
    out = ctx.forward_batch(MiniBatch.prefill(slots, [s[:h] for s, h in zip(seqs, heads)]))
    for i, h in enumerate(heads):
        assert err(out[i], want[i][h - 1]) <= tol
    live = list(range(3))
    t = 0
    while live:
        out = ctx.forward_batch(MiniBatch.decode([slots[i] for i in live], [seqs[i][heads[i] + t] for i in live]))
        for row, i in enumerate(live):
            assert err(out[row], want[i][heads[i] + t]) <= tol
        t += 1
        for i in [i for i in live if heads[i] + t == len(seqs[i])]:
            ctx.release(slots[i])
        live = [i for i in live if heads[i] + t < len(seqs[i])]
    cache.check()
    assert llm.generate([[1, 2, 3]], n_predict=4, stop_token_ids=[])[0].__len__() == 4


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_stateful_mixer_that_may_be_captured_advances_its_state_once_a_step(dtype, tmp_path):
    """Steps through a mixer that declares itself `graph_safe` are captured into CUDA graphs, and a capture is preceded
    by an eager warm-up run of the same step (`DecodeRunner.capture`, `Context._forward_maybe_replayed`).  Keys and
    values land on the same places both times; fixed-size state would be advanced twice unless the warm-up run's
    state is put back (`PagedCache.snapshot_state`).  Every step's logits are compared with the plain recurrence."""
    folder = ml.write_random_model(ModelConfig.from_dict(dict(RAW, toy_kind="toy_decay_on_device")), str(tmp_path / "toy"), 7, std=0.1)
    llm = ml.load(folder, dtype=dtype, max_tokens=2048, max_seqs=4)
    assert llm.context.use_graphs
    tol = 2e-5 if dtype == "float32" else 3e-2
    prompts = [helpers.random_tokens(n, 200, 30 + n) for n in (9, 2, 17)]
    seen = []
    out = llm.generate(prompts, n_predict=20, temperature=1.0, seed=5, stop_token_ids=[],
                       on_step=lambda live, chosen, logits: seen.append((list(live), logits.float().cpu().clone())))
    refs = [plain_logits(folder, p + o) for p, o in zip(prompts, out)]
    for k, (live, logits) in enumerate(seen):
        for row, i in enumerate(live):
            ref = refs[i][len(prompts[i]) - 1 + k]
            assert float((logits[row].double() - ref.double()).abs().max() / ref.abs().max()) <= tol, (k, i)
    # a prompt step of a shape that comes again: issued kernel by kernel the first time, warmed up and captured the
    # second, replayed the third; each time followed by one decoded token that reads the state the step left
    ctx = llm.context
    for round_ in range(3):
        seqs = [helpers.random_tokens(n, 200, 60 + 10 * round_ + n) for n in (70, 40)]
        slots = [ctx.acquire() for _ in seqs]
        got = ctx.forward_batch(MiniBatch.prefill(slots, seqs))
        nxt = ctx.forward_batch(MiniBatch.decode(slots, [3, 4]))
        for i, toks in enumerate(seqs):
            ref = plain_logits(folder, toks + [3 + i])
            assert float((got[i].double().cpu() - ref[-2].double()).abs().max() / ref[-2].abs().max()) <= tol, (round_, i)
            assert float((nxt[i].double().cpu() - ref[-1].double()).abs().max() / ref[-1].abs().max()) <= tol, (round_, i)
        for s_ in slots:
            ctx.release(s_)
    assert len(ctx._step_graphs) == 1
    ctx.cache.check()
