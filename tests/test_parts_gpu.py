"""Each part alone against the plain implementation's function for it, built through the
part registry with sizes other than the engine tests', and a model whose schedule runs a
layer twice and lets a run read another run's cache."""
import math

import pytest
import torch

import helpers
import plain_impl
from mini_llama_cpp_release_b200.cache import PagedCache
from mini_llama_cpp_release_b200.config import ModelConfig, PartSpec, ScheduleEntry, build_part, register_architecture
from mini_llama_cpp_release_b200.config.specs import ModelSpec
from mini_llama_cpp_release_b200.engine import Context, MiniBatch, Model
from mini_llama_cpp_release_b200.engine.batch import SequenceChunk
from mini_llama_cpp_release_b200.models.qwen2 import Qwen2Config, qwen2
from mini_llama_cpp_release_b200.parts import MixerMemory, Runtime
from mini_llama_cpp_release_b200.weights.random_init import random_tensor

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 5e-6, "bfloat16": 2e-2}


def bound(spec: PartSpec, name: str, dtype: str, seed=0, std=0.3):
    """Build a part, give it random tensors; returns (part, {name: float32 cpu tensor})."""
    part = build_part(spec, name)
    rt = Runtime(DEV, DT[dtype])
    tensors = {s.name: random_tensor(s, seed, DT[dtype], std=std) for s in part.all_tensors()}
    part.bind(lambda n: tensors[n].to(DEV) if n in tensors else None, rt)
    return part, {k: v.float() for k, v in tensors.items()}


def close(got, want, tol):
    err = float((got.double().cpu() - want.double()).abs().max() / want.double().abs().max().clamp_min(1e-30))
    assert err <= tol, err


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_norm_part(dtype):
    norm, w = bound(PartSpec("norm", "rmsnorm", dict(size=200, eps=3e-4)), "n.", dtype)
    x, d = torch.randn(6, 200) * 2, torch.randn(6, 200)
    xd = x.to(DEV)
    h = norm.forward(xd, d.to(DEV))
    close(h.float(), plain_impl.rmsnorm(x + d, w["n.weight"], 3e-4), TOL[dtype])
    close(xd, x + d, 1e-6)
    assert h.dtype == DT[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_position_part(dtype):
    rope, _ = bound(PartSpec("position", "rope_neox", dict(head_dim=48, theta=12345.0, max_positions=4096)), "p.", dtype)
    x = torch.randn(5, 3, 48)
    pos = torch.tensor([0, 1, 77, 1000, 4095], dtype=torch.int32)
    got = rope.rotate(x.to(DEV), pos.to(DEV))
    close(got.float(), plain_impl.rope_neox(x, pos, 12345.0), TOL[dtype])
    with pytest.raises(ValueError, match="even"):
        build_part(PartSpec("position", "rope_neox", dict(head_dim=15, theta=1e4, max_positions=8)), "p.")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_feed_forward_part(dtype):
    ffn, w = bound(PartSpec("feed_forward", "swiglu", dict(hidden_size=72, intermediate_size=100)), "m.", dtype)
    h = torch.randn(9, 72).to(DT[dtype])
    got = ffn.forward(h.to(DEV))
    got = got.sum(0) if got.dim() == 3 else got
    want = plain_impl.swiglu_ffn(h.float(), w["m.gate_proj.weight"], w["m.up_proj.weight"], w["m.down_proj.weight"])
    close(got, want, TOL[dtype])
    assert got.dtype == torch.float32
    with pytest.raises(ValueError, match="silu"):
        build_part(PartSpec("feed_forward", "swiglu", dict(hidden_size=8, intermediate_size=8, activation="relu")), "m.")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embedding_and_head_parts(dtype):
    emb, w = bound(PartSpec("embedding", "token_embedding", dict(vocab_size=301, hidden_size=40)), "e.", dtype)
    ids = torch.tensor([300, 0, 7], dtype=torch.int32)
    assert torch.equal(emb.forward(ids.to(DEV)).cpu(), w["e.weight"][ids.long()])
    head, hw = bound(PartSpec("head", "linear_head", dict(vocab_size=301, hidden_size=40)), "h.", dtype)
    h = torch.randn(4, 40).to(DT[dtype])
    close(head.forward(h.to(DEV)), h.float() @ hw["h.weight"].t(), TOL[dtype])
    tied = build_part(PartSpec("head", "linear_head", dict(vocab_size=301, hidden_size=40, tied_to="e.weight")), "h.")
    tied.bind(lambda n: emb.table if n == "e.weight" else None, emb.runtime)
    assert tied.proj.weight.data_ptr() == emb.table.data_ptr()                  # an alias, not a copy
    assert [s.stored for s in tied.tensors()] == [False]


def attention_spec(H, KV, hd, hidden, window=None, bias=True, theta=1e4):
    rope = PartSpec("position", "rope_neox", dict(head_dim=hd, theta=theta, max_positions=2048))
    return PartSpec("mixer", "gqa_attention", dict(hidden_size=hidden, num_heads=H, num_kv_heads=KV, head_dim=hd,
                                                   qkv_bias=bias, position=rope, window=window))


def run_mixer(att, dtype, hs, splits):
    """Feed each sequence's rows h [T, hidden] through the mixer in the given cuts, with a
    cache of its own; returns per-sequence outputs [T, hidden]."""
    cache = PagedCache([att.cache_need()], [None], [None], 64 * 40, 8, DT[dtype], DEV)
    from mini_llama_cpp_release_b200.engine.context import Context

    class Shim:                      # the few things Context.describe needs
        pass
    ctx = Context.__new__(Context)
    ctx.cache, ctx.max_position = cache, 4096
    ctx.model = Shim(); ctx.model.runtime = att.runtime
    slots = [cache.acquire() for _ in hs]
    done = [0] * len(hs)
    outs = [[] for _ in hs]
    for cut in splits:                # cut: how many tokens each sequence brings to this step (0: none)
        chunks, rows = [], []
        for b, n in enumerate(cut):
            if n:
                chunks.append(SequenceChunk(slots[b], [0] * n, []))
                rows.append(hs[b][done[b]:done[b] + n])
        step = ctx.describe(MiniBatch(chunks))
        y = att.forward(torch.cat(rows).to(DT[dtype]).to(DEV), step, MixerMemory(kv=cache.view(0, step.page_tables)))
        y = y.sum(0) if y.dim() == 3 else y          # a branch may leave split-K partial sums for the next norm to add
        off = 0
        for b, n in enumerate(cut):
            if n:
                outs[b].append(y[off:off + n].float().cpu()); off += n
                cache.commit(slots[b], n); done[b] += n
    return [torch.cat(o) for o in outs]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,KV,hd,window,bias", [(6, 3, 32, None, True), (14, 2, 64, None, True), (4, 1, 16, 20, False)])
def test_attention_part_whole_chunked_and_batched(H, KV, hd, window, bias, dtype):
    hidden = 72
    att, w = bound(attention_spec(H, KV, hd, hidden, window, bias), "a.", dtype, std=0.2)
    hs = [torch.randn(n, hidden).to(DT[dtype]).float() for n in (70, 9, 1)]
    cfg = dict(num_attention_heads=H, num_key_value_heads=KV, head_dim=hd, rope_theta=1e4)
    want = [plain_impl.attention_block(h, {k.replace("a.", "p.self_attn."): v for k, v in w.items()}, "p.", cfg,
                                       torch.arange(len(h)), window) for h in hs]
    whole = run_mixer(att, dtype, hs, [[70, 9, 1]])
    cuts = run_mixer(att, dtype, hs, [[60, 5, 0], [1, 1, 1], [9, 3, 0]])
    for a, b, c in zip(whole, cuts, want):
        close(a, c, TOL[dtype])
        close(b, c, TOL[dtype])


def twice_and_shared(config: ModelConfig) -> ModelSpec:
    """Qwen2's parts under another schedule: layer 0, layer 1, layer 0 again (a cache of its
    own), then layer 1 reading the cache its first run wrote."""
    base = qwen2(config)
    return ModelSpec(base.config, base.embedding, base.layers,
                     (ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0), ScheduleEntry(1, reads_cache_of=1)),
                     base.final_norm, base.head)


def plain_twice_and_shared(cfg, w, tokens):
    x = plain_impl.embedding(w["model.embed_tokens.weight"], tokens)
    pos = torch.arange(len(tokens))
    H, KV, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    kept = {}
    for run, (layer, shared) in enumerate([(0, None), (1, None), (0, None), (1, 1)]):
        p = f"model.layers.{layer}."
        h = plain_impl.rmsnorm(x, w[p + "input_layernorm.weight"], cfg["rms_norm_eps"])
        T = len(tokens)
        q = plain_impl.linear(h, w[p + "self_attn.q_proj.weight"], w[p + "self_attn.q_proj.bias"])
        q = plain_impl.rope_neox(q.view(T, H, hd), pos, cfg["rope_theta"])
        if shared is None:
            k = plain_impl.linear(h, w[p + "self_attn.k_proj.weight"], w[p + "self_attn.k_proj.bias"])
            v = plain_impl.linear(h, w[p + "self_attn.v_proj.weight"], w[p + "self_attn.v_proj.bias"])
            k = plain_impl.rope_neox(k.view(T, KV, hd), pos, cfg["rope_theta"])
            kept[run] = (k, v.view(T, KV, hd))
        k, v = kept[run if shared is None else shared]
        o = plain_impl.attention(q, k, v)
        x = x + plain_impl.linear(o.reshape(T, H * hd), w[p + "self_attn.o_proj.weight"])
        h2 = plain_impl.rmsnorm(x, w[p + "post_attention_layernorm.weight"], cfg["rms_norm_eps"])
        x = x + plain_impl.swiglu_ffn(h2, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    h = plain_impl.rmsnorm(x, w["model.norm.weight"], cfg["rms_norm_eps"])
    return plain_impl.linear(h, w["model.embed_tokens.weight"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_schedule_runs_a_layer_twice_and_shares_a_cache(dtype, tmp_path):
    import mini_llama_cpp_release_b200 as ml
    register_architecture("TwiceAndShared", config_class=Qwen2Config)(twice_and_shared)      # Qwen2's keys, another schedule
    raw = dict(helpers.TINY_A, architectures=["TwiceAndShared"])
    folder = ml.write_random_model(ModelConfig.from_dict(raw), str(tmp_path / "m"), 3, std=0.1)
    llm = ml.load(folder, dtype=dtype, max_tokens=1024)
    assert len(llm.context.cache.groups) == 1 and llm.context.cache.groups[0].entries == [0, 1, 2]
    assert llm.context.cache.where[3] == llm.context.cache.where[1]
    toks = helpers.random_tokens(80, 512, 1)
    want = plain_twice_and_shared(plain_impl.read_config(folder), plain_impl.read_weights(folder), toks)
    ctx = llm.context
    s = ctx.acquire()
    got = [ctx.forward_batch(MiniBatch.from_tokens(s, toks[:70], want=list(range(70))))]
    got += [ctx.forward_batch(MiniBatch.single(s, t)) for t in toks[70:]]
    ctx.release(s)
    tol = 2e-5 if dtype == "float32" else 3e-2
    close(torch.cat(got), want, tol)
