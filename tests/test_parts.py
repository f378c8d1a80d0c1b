"""Each part of the decoder alone, on the GPU, against the plain function of the same name,
driven through a real step context (cache pages, slots, block tables) of a model whose sizes
differ from both tiny configurations."""

from __future__ import annotations

import pytest
import torch

import helpers
import plain_llama as plain

pytestmark = pytest.mark.gpu

RAW = {
    "architectures": ["LlamaForCausalLM"], "num_hidden_layers": 2, "hidden_size": 80, "num_attention_heads": 6,
    "num_key_value_heads": 2, "head_dim": 48, "intermediate_size": 112, "vocab_size": 333, "rope_theta": 30000.0,
    "rms_norm_eps": 2e-5, "tie_word_embeddings": False, "max_position_embeddings": 4096,
}


def tol(dtype):
    return dict(atol=3e-5, rtol=3e-5) if dtype == "float32" else dict(atol=3e-2, rtol=3e-2)


def assert_close_scaled(got, want, dtype):
    """float32: elementwise; bfloat16: the suite's rule for whole-layer outputs, an error bounded by
    a fraction of the output's scale (helpers.BF16_FRACTION / BF16_MEAN_FRACTION)."""
    import helpers

    if dtype == "float32":
        torch.testing.assert_close(got, want, atol=3e-5, rtol=3e-5)
        return
    err, scale = (got - want).abs(), float(want.abs().max())
    assert float(err.max()) <= helpers.BF16_FRACTION * scale, (float(err.max()), scale)
    assert float(err.mean()) <= helpers.BF16_MEAN_FRACTION * scale, (float(err.mean()), scale)


@pytest.fixture(scope="module", params=["float32", "bfloat16"])
def rig(request, tmp_path_factory):
    from edgerag_b200.engine.engine import Engine

    dtype = request.param
    folder = plain.write_model_folder(tmp_path_factory.mktemp("parts") / dtype, RAW, seed=5, std=0.15,
                                      dtype=getattr(torch, dtype))
    engine = Engine.from_pretrained(folder, dtype=dtype, block_size=8, num_blocks=40, max_batch_size=4,
                                    chunk_size=64, poison_freed_pages=True)
    return dtype, engine, plain.read_config(folder), plain.read_weights(folder)


def context(engine, n_tokens=19, rid="r"):
    from edgerag_b200.engine.step import StepEntry

    runner = engine.runner
    if rid in runner.cache.requests:
        runner.release(rid)
    runner.admit(rid)
    ids = torch.randint(0, RAW["vocab_size"], (n_tokens,), generator=torch.Generator().manual_seed(1)).tolist()
    ctx, ordered = runner.prepare([StepEntry(rid, tokens=ids, want=[0, n_tokens - 1])])
    return ctx, ordered, ids


def test_embedding_norm_and_head(rig):
    dtype, engine, cfg, w = rig
    model = engine.model
    ctx, ordered, ids = context(engine)
    hidden = torch.empty((len(ids), cfg["hidden"]), device="cuda")
    model.embedding.forward(ctx, hidden)
    want_h = plain.embed(w, torch.tensor(ids))
    assert torch.equal(hidden.cpu(), want_h)
    out = torch.empty((len(ids), cfg["hidden"]), dtype=model.dtype, device="cuda")
    model.final_norm.forward(hidden, out)
    want_n = plain.rms_norm(want_h, w["model.norm.weight"], cfg["eps"])
    torch.testing.assert_close(out.float().cpu(), want_n, **tol(dtype))
    logits = torch.empty((len(ids), cfg["vocab"]), device="cuda")
    model.head.forward(out, logits)
    torch.testing.assert_close(logits.cpu(), out.float().cpu() @ w["lm_head.weight"].T, **tol(dtype))
    engine.runner.finish(ordered)


def test_attention_mixer_whole_and_continued(rig):
    """The mixer over a fresh sequence, then over a continuation that reads the first part from the cache."""
    dtype, engine, cfg, w = rig
    from edgerag_b200.engine.step import StepEntry

    mixer = engine.model.blocks[1].mixer
    call = engine.model.schedule[1]
    runner = engine.runner
    if "m" in runner.cache.requests:
        runner.release("m")
    runner.admit("m")
    n1, n2 = 21, 13
    x_all = (0.5 * torch.randn((n1 + n2, cfg["hidden"]), generator=torch.Generator().manual_seed(2))).to(engine.dtype)
    p = "model.layers.1.self_attn."
    want = plain.attention(x_all.float(), torch.arange(n1 + n2), w[p + "q_proj.weight"], w[p + "k_proj.weight"],
                           w[p + "v_proj.weight"], w[p + "o_proj.weight"], cfg)
    got = []
    for lo, hi in ((0, n1), (n1, n1 + n2)):
        ctx, ordered = runner.prepare([StepEntry("m", tokens=[1] * (hi - lo))])
        got.append(helpers.whole_update(mixer.forward(x_all[lo:hi].cuda().contiguous(), ctx, call)).cpu())
        runner.finish(ordered)
    assert_close_scaled(torch.cat(got), want, dtype)
    # one more token: the decode kernel's path
    ctx, ordered = runner.prepare([StepEntry("m", tokens=[1])])
    x_new = (0.5 * torch.randn((1, cfg["hidden"]), generator=torch.Generator().manual_seed(3))).to(engine.dtype)
    y = helpers.whole_update(mixer.forward(x_new.cuda(), ctx, call)).cpu()
    runner.finish(ordered)
    full = plain.attention(torch.cat([x_all, x_new]).float(), torch.arange(n1 + n2 + 1), w[p + "q_proj.weight"],
                           w[p + "k_proj.weight"], w[p + "v_proj.weight"], w[p + "o_proj.weight"], cfg)
    assert_close_scaled(y, full[-1:], dtype)
    runner.release("m")


def test_feed_forward(rig):
    dtype, engine, cfg, w = rig
    ffn = engine.model.blocks[0].ffn
    ctx, ordered, ids = context(engine, 7)
    x = torch.randn((7, cfg["hidden"]), generator=torch.Generator().manual_seed(4)).to(engine.dtype)
    p = "model.layers.0.mlp."
    want = plain.swiglu(x.float(), w[p + "gate_proj.weight"], w[p + "up_proj.weight"], w[p + "down_proj.weight"])
    got = helpers.whole_update(ffn.forward(x.cuda(), ctx)).cpu()
    assert_close_scaled(got, want, dtype)
    engine.runner.finish(ordered)


def test_block_arrangement(rig):
    """A whole pre-norm block: hidden and pending update together equal the plain layer's output."""
    dtype, engine, cfg, w = rig
    block = engine.model.blocks[0]
    ctx, ordered, ids = context(engine, 23, rid="blk")
    h0 = torch.randn((23, cfg["hidden"]), generator=torch.Generator().manual_seed(6))
    hidden = h0.clone().cuda()
    delta = block.forward(hidden, None, ctx, engine.model.schedule[0])
    want = plain.decoder_layer(h0, torch.arange(23), w, 0, cfg)
    assert_close_scaled((hidden + helpers.whole_update(delta)).cpu(), want, dtype)
    engine.runner.finish(ordered)
    engine.runner.release("blk")


def test_position_encoding_part(rig):
    dtype, engine, cfg, w = rig
    from edgerag_b200.parts.base import PartSpec, build_part

    rope = build_part("position", PartSpec("rope_halves", {"head_dim": 48, "theta": 30000.0}), engine.dtype, engine.device)
    ctx, ordered, ids = context(engine, 9, rid="pe")
    qkv = torch.randn((9, (6 + 4) * 48), generator=torch.Generator().manual_seed(8)).to(engine.dtype).cuda()
    before = qkv.float().cpu().view(9, 10, 48)
    rope.apply_and_store(qkv, ctx, 6, 2, 48, None, None)       # no pages: only q is rotated, in place
    cos, sin = plain.rope_tables(torch.arange(9), 48, 30000.0)
    want_q = plain.apply_rope(before[:, :6].transpose(0, 1), cos, sin).transpose(0, 1)
    got = qkv.float().cpu().view(9, 10, 48)
    torch.testing.assert_close(got[:, :6], want_q.to(engine.dtype).float(), **tol(dtype))
    assert torch.equal(got[:, 6:], before[:, 6:])
    none = build_part("position", PartSpec("none"), engine.dtype, engine.device)
    k_pages, v_pages = ctx.pages_of(0)
    none.apply_and_store(qkv, ctx, 6, 2, 48, (k_pages, v_pages), ctx.slots[0])
    slot = int(ctx.slots[0][4])
    assert torch.equal(k_pages[slot // 8, :, slot % 8].float().cpu(), got[4, 6:8])   # stored as is
    engine.runner.finish(ordered)
    engine.runner.release("pe")
