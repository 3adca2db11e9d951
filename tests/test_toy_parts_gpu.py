"""A feed-forward with routing and another position encoding, both defined here, are registered,
built, given random weights, loaded and stepped through the library's public hooks alone.

The toy feed-forward sends each token to the one expert whose router logit is largest and
weights that expert's output with the softmax probability of the choice.  The toy position
encoding rotates only the first `n_rotated` pairs of a head, by angles of a stretched position
(p / stretch); the other pairs are left as they are.  The toy architecture uses them in its
first layer and the library's own rotation and feed-forward in its second, so one model has
different feed-forwards and position encodings in different layers."""
import pytest
import torch

import helpers
import plain_impl
import mini_llama_cpp_release_b200 as ml
from mini_llama_cpp_release_b200.config import ModelConfig, ModelSpec, PartSpec, prenorm_layer, sequential_schedule
from mini_llama_cpp_release_b200.engine import MiniBatch
from mini_llama_cpp_release_b200.models.qwen2 import LAYER_NAMES
from mini_llama_cpp_release_b200.parts import Part, TensorSpec

pytestmark = pytest.mark.gpu


def toy_angles(head_dim, theta, n_rotated, stretch, n_positions):
    """[n_positions, head_dim/2] float32 angles: (p / stretch) * theta^(-2i/hd) for pair i < n_rotated, else 0."""
    i = torch.arange(head_dim // 2, dtype=torch.float32)
    freq = torch.where(i < n_rotated, torch.pow(torch.tensor(float(theta)), -2.0 * i / head_dim), torch.zeros(()))
    return (torch.arange(n_positions, dtype=torch.float32) / stretch)[:, None] * freq[None, :]


@ml.register_part("position", "toy_partial_stretched")
class ToyPartialStretchedRotation(Part):
    graph_safe = True
    fusable = True          # a table of cos and sin per position and pair is all the attention part needs

    def __init__(self, name, head_dim, theta, n_rotated, stretch, max_positions):
        super().__init__(name, head_dim=head_dim, theta=theta, n_rotated=n_rotated, stretch=stretch, max_positions=max_positions)
        self.head_dim, self.theta, self.n_rotated, self.stretch, self.max_positions = head_dim, theta, n_rotated, stretch, max_positions
        self.table = None

    def prepare(self, n_positions):
        if self.table is None:
            a = toy_angles(self.head_dim, self.theta, self.n_rotated, self.stretch, self.max_positions)
            self.table = torch.stack([torch.cos(a), torch.sin(a)], dim=-1).contiguous().to(self.runtime.device)


@ml.register_part("feed_forward", "toy_routed")
class ToyRoutedFeedForward(Part):
    def __init__(self, name, hidden_size, expert_size, n_experts):
        super().__init__(name, hidden_size=hidden_size, expert_size=expert_size, n_experts=n_experts)
        self.hidden, self.inner, self.E = hidden_size, expert_size, n_experts

    def tensors(self):
        specs = [TensorSpec(self.name + "router.weight", (self.E, self.hidden))]
        for e in range(self.E):
            specs += [TensorSpec(self.name + f"experts.{e}.up.weight", (self.inner, self.hidden)),
                      TensorSpec(self.name + f"experts.{e}.down.weight", (self.hidden, self.inner))]
        return specs

    def bind(self, get, runtime):
        super().bind(get, runtime)
        self.router = get(self.name + "router.weight").float()
        self.up = torch.stack([get(self.name + f"experts.{e}.up.weight").float() for e in range(self.E)])
        self.down = torch.stack([get(self.name + f"experts.{e}.down.weight").float() for e in range(self.E)])

    def forward(self, h, step=None):
        h = h.float()
        logits = h @ self.router.t()                                   # float32 router logits
        prob, choice = torch.softmax(logits, dim=-1).max(dim=-1)
        inner = torch.relu(torch.einsum("nh,nih->ni", h, self.up[choice]))
        return torch.einsum("ni,nhi->nh", inner, self.down[choice]) * prob[:, None]


@ml.register_architecture("ToyRoutedLM")
def toy_routed_lm(c: ModelConfig) -> ModelSpec:
    norm = PartSpec("norm", "rmsnorm", dict(size=c.hidden_size, eps=c.rms_norm_eps))
    rope = PartSpec("position", "rope_neox", dict(head_dim=c.head_dim, theta=c.rope_theta, max_positions=c.max_position_embeddings))
    toy_pos = PartSpec("position", "toy_partial_stretched",
                       dict(head_dim=c.head_dim, theta=c.rope_theta, n_rotated=c.extra["toy_n_rotated"],
                            stretch=c.extra["toy_stretch"], max_positions=c.max_position_embeddings))

    def attn(position):
        return PartSpec("mixer", "gqa_attention", dict(hidden_size=c.hidden_size, num_heads=c.num_attention_heads,
                                                       num_kv_heads=c.num_key_value_heads, head_dim=c.head_dim, qkv_bias=True,
                                                       position=position))
    swiglu = PartSpec("feed_forward", "swiglu", dict(hidden_size=c.hidden_size, intermediate_size=c.intermediate_size))
    routed = PartSpec("feed_forward", "toy_routed", dict(hidden_size=c.hidden_size, expert_size=c.extra["toy_expert_size"],
                                                         n_experts=c.extra["toy_n_experts"]))
    layers = (prenorm_layer("model.layers.0.", attn(toy_pos), routed, norm, norm, LAYER_NAMES),
              prenorm_layer("model.layers.1.", attn(rope), swiglu, norm, norm, LAYER_NAMES))
    return ModelSpec(c, PartSpec("embedding", "token_embedding", dict(vocab_size=c.vocab_size, hidden_size=c.hidden_size)),
                     layers, sequential_schedule(len(layers)), norm,
                     PartSpec("head", "linear_head", dict(vocab_size=c.vocab_size, hidden_size=c.hidden_size)))


RAW = dict(architectures=["ToyRoutedLM"], hidden_size=64, intermediate_size=88, num_hidden_layers=2, num_attention_heads=4,
           num_key_value_heads=2, head_dim=32, vocab_size=150, max_position_embeddings=128, rope_theta=1e4,
           rms_norm_eps=1e-5, toy_n_rotated=10, toy_stretch=4.0, toy_expert_size=24, toy_n_experts=3)
LENGTHS = (12, 5, 9)


def toy_rotate(x, positions):
    hd, half = RAW["head_dim"], RAW["head_dim"] // 2
    a = toy_angles(hd, RAW["rope_theta"], RAW["toy_n_rotated"], RAW["toy_stretch"], 128)[positions][:, None, :]
    lo, hi = x[..., :half], x[..., half:]
    return torch.cat([lo * torch.cos(a) - hi * torch.sin(a), lo * torch.sin(a) + hi * torch.cos(a)], dim=-1)


def plain_logits(folder, tokens):
    """Logits of one whole sequence and the smallest gap between the two largest router logits, relative to the largest
    logit in size: how far the routing decisions are from a tie."""
    cfg, w = plain_impl.read_config(folder), plain_impl.read_weights(folder)
    H, KV, hd, T = 4, 2, 32, len(tokens)
    x = plain_impl.embedding(w["model.embed_tokens.weight"], tokens)
    pos = torch.arange(T)
    # layer 0: attention with the toy rotation, routed feed-forward
    p = "model.layers.0."
    h = plain_impl.rmsnorm(x, w[p + "input_layernorm.weight"], 1e-5)
    q = plain_impl.linear(h, w[p + "self_attn.q_proj.weight"], w[p + "self_attn.q_proj.bias"]).view(T, H, hd)
    k = plain_impl.linear(h, w[p + "self_attn.k_proj.weight"], w[p + "self_attn.k_proj.bias"]).view(T, KV, hd)
    v = plain_impl.linear(h, w[p + "self_attn.v_proj.weight"], w[p + "self_attn.v_proj.bias"]).view(T, KV, hd)
    o = plain_impl.attention(toy_rotate(q, pos), toy_rotate(k, pos), v, None)
    x = x + plain_impl.linear(o.reshape(T, H * hd), w[p + "self_attn.o_proj.weight"])
    h2 = plain_impl.rmsnorm(x, w[p + "post_attention_layernorm.weight"], 1e-5)
    logits = h2 @ w[p + "mlp.router.weight"].t()
    top = logits.topk(2, dim=-1).values
    margin = float(((top[:, 0] - top[:, 1]) / logits.abs().max(dim=-1).values).min())
    rows = []
    for t in range(T):
        e = int(logits[t].argmax())
        inner = torch.relu(w[p + f"mlp.experts.{e}.up.weight"] @ h2[t])
        rows.append(w[p + f"mlp.experts.{e}.down.weight"] @ inner * torch.softmax(logits[t], dim=-1)[e])
    x = x + torch.stack(rows)
    # layer 1: the library's own parts
    x = plain_impl.decoder_layer(x, w, 1, cfg, pos)
    return plain_impl.linear(plain_impl.rmsnorm(x, w["model.norm.weight"], 1e-5), w["lm_head.weight"]), margin


def model_whose_routing_is_clear(tmp_path, least_margin):
    """Random weights whose routing decisions, on the test's sequences, are not within rounding of a tie: a decision that
    bfloat16 activations could turn would compare two different experts and say nothing about the parts."""
    for seed in range(40):
        folder = ml.write_random_model(ModelConfig.from_dict(RAW), str(tmp_path / f"toy{seed}"), seed, std=0.15)
        seqs = [helpers.random_tokens(n, 150, n + seed) for n in LENGTHS]
        plain = [plain_logits(folder, s) for s in seqs]
        if min(m for _, m in plain) >= least_margin:
            return folder, seqs, [l for l, _ in plain]
    raise AssertionError("no seed gives clear routing decisions")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_feed_forward_with_routing_and_toy_position_encoding_register_build_and_step(dtype, tmp_path):
    folder, seqs, want = model_whose_routing_is_clear(tmp_path, 1e-3 if dtype == "float32" else 0.1)
    llm = ml.load(folder, dtype=dtype, max_tokens=1024, max_seqs=4)
    ctx = llm.context
    tol = 2e-5 if dtype == "float32" else 3e-2

    def err(got, ref):
        return float((got.double().cpu() - ref.double()).abs().max() / ref.abs().max())

    for s, ref in zip(seqs, want):                                  # whole, each alone
        slot = ctx.acquire()
        assert err(ctx.forward_batch(MiniBatch.from_tokens(slot, s, want=list(range(len(s))))), ref) <= tol
        ctx.release(slot)
    slots = [ctx.acquire() for _ in seqs]                           # prompts of unequal length, then one token each
    heads = [4, 1, 8]
    out = ctx.forward_batch(MiniBatch.prefill(slots, [s[:h] for s, h in zip(seqs, heads)]))
    for i, h in enumerate(heads):
        assert err(out[i], want[i][h - 1]) <= tol
    live, t = list(range(3)), 0
    while live:
        out = ctx.forward_batch(MiniBatch.decode([slots[i] for i in live], [seqs[i][heads[i] + t] for i in live]))
        for row, i in enumerate(live):
            assert err(out[row], want[i][heads[i] + t]) <= tol
        t += 1
        for i in [i for i in live if heads[i] + t == len(seqs[i])]:
            ctx.release(slots[i])
        live = [i for i in live if heads[i] + t < len(seqs[i])]
    ctx.cache.check()
    assert len(llm.generate([[1, 2, 3]], n_predict=4, stop_token_ids=[])[0]) == 4


def test_the_toy_position_encoding_differs_from_the_librarys_own(tmp_path):
    """The comparison above would pass with the library's rotation in both layers if the two agreed: they do not."""
    x = torch.randn(6, 2, 32)
    pos = torch.arange(6) + 40
    assert (toy_rotate(x, pos) - plain_impl.rope_neox(x, pos, 1e4)).abs().max() > 0.1
