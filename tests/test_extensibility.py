"""Parts and architectures are added from outside: a toy mixer with state of its own, defined
here, is registered, built into a model by a plan, loaded from a folder and stepped, portion by
portion and beside other requests, without a change to the framework's files."""

from __future__ import annotations

import json

import pytest
import torch

pytestmark = pytest.mark.gpu

HIDDEN, VOCAB, LAYERS = 48, 97, 3
DECAY = 0.9


def register_toy():
    from edgerag_b200.cache.manager import StateSpec
    from edgerag_b200.config import register_architecture
    from edgerag_b200.parts.base import (LayerCall, LayerSpec, Mixer, ModelPlan, PartSpec, WeightSpec,
                                         register_part)

    @register_part("mixer", "toy_decay")
    class ToyDecayMixer(Mixer):
        """y_t = W (s_t),  s_t = decay * s_{t-1} + x_t: a running state of fixed size per request."""

        def __init__(self, hidden, decay, dtype, device):
            self.hidden, self.decay, self.dtype, self.device = hidden, decay, dtype, device
            self.w = None

        def cache_spec(self):
            return [StateSpec("toy_state", (self.hidden,), "float32")]

        def weight_specs(self):
            return [WeightSpec("mix.weight", (self.hidden, self.hidden))]

        def load_weights(self, tensors):
            self.w = tensors["mix.weight"].to(device=self.device, dtype=self.dtype)

        def forward(self, x, ctx, call):
            from edgerag_b200.ops import kernels

            state = ctx.state("toy_state", call.cache_layer)         # [slots, hidden]
            out = ctx.buf("toy.s", (x.shape[0], self.hidden), self.dtype)
            t0 = 0
            for s, n in enumerate(ctx.host_q_len):                    # each request's slot is updated once per step
                slot = ctx.host_state_slots[s]
                cur = state[slot]
                for t in range(t0, t0 + n):
                    cur = self.decay * cur + x[t].float()
                    out[t] = cur.to(self.dtype)
                state[slot] = cur
                t0 += n
            y = ctx.buf("toy.y", (x.shape[0], self.hidden), self.dtype)
            kernels.linear(out, self.w, y)
            return y

    def read_config(raw, where):
        return raw

    def make_plan(raw):
        h = raw["hidden_size"]
        norm = lambda p: PartSpec("rmsnorm", {"size": h, "eps": raw["eps"]}, p)   # noqa: E731
        layers = []
        for i in range(raw["num_hidden_layers"]):
            if i % 2 == 0:
                mixer = PartSpec("toy_decay", {"hidden": h, "decay": raw["decay"]}, "toy.")
            else:   # a different mixer in a different layer of the same model
                mixer = PartSpec("attention", {"hidden": h, "n_q_heads": 2, "n_kv_heads": 1, "head_dim": 16,
                                               "position": PartSpec("rope_halves", {"head_dim": 16, "theta": 1000.0})}, "self_attn.")
            layers.append(LayerSpec(f"layers.{i}.", PartSpec("prenorm"), norm("ln1."), mixer, norm("ln2."),
                                    PartSpec("swiglu", {"hidden": h, "intermediate": 2 * h}, "mlp.")))
        return ModelPlan(h, raw["vocab_size"], PartSpec("table", {"vocab": raw["vocab_size"], "hidden": h}, "embed_tokens."),
                         layers, [LayerCall(i, i) for i in range(len(layers))], norm("norm."),
                         PartSpec("linear", {"vocab": raw["vocab_size"], "hidden": h, "tied_to": "embed_tokens.weight"}, "lm_head."))

    register_architecture("ToyDecayForCausalLM", read_config, make_plan)


def plain_toy(weights, raw, ids):
    """Whole-sequence float32 computation of the toy model, written out with no engine code."""
    import plain_llama as plain

    h = weights["model.embed_tokens.weight"][torch.tensor(ids)]
    n = h.shape[0]
    for i in range(raw["num_hidden_layers"]):
        p = f"model.layers.{i}."
        x = plain.rms_norm(h, weights[p + "ln1.weight"], raw["eps"])
        if i % 2 == 0:
            s, rows = torch.zeros(raw["hidden_size"]), []
            for t in range(n):
                s = raw["decay"] * s + x[t]
                rows.append(s)
            h = h + torch.stack(rows) @ weights[p + "toy.mix.weight"].T
        else:
            cfg = {"head_dim": 16, "n_q": 2, "n_kv": 1, "theta": 1000.0}
            a = p + "self_attn."
            h = h + plain.attention(x, torch.arange(n), weights[a + "q_proj.weight"], weights[a + "k_proj.weight"],
                                    weights[a + "v_proj.weight"], weights[a + "o_proj.weight"], cfg)
        y = plain.rms_norm(h, weights[p + "ln2.weight"], raw["eps"])
        m = p + "mlp."
        h = h + plain.swiglu(y, weights[m + "gate_proj.weight"], weights[m + "up_proj.weight"], weights[m + "down_proj.weight"])
    return plain.rms_norm(h, weights["model.norm.weight"], raw["eps"]) @ weights["model.embed_tokens.weight"].T


def test_toy_mixer_with_state_is_registered_built_and_stepped(tmp_path):
    register_toy()
    from edgerag_b200 import Engine
    from edgerag_b200.config.registry import architecture_of
    from edgerag_b200.engine.step import StepEntry
    from edgerag_b200.models.decoder import DecoderModel
    from edgerag_b200.weights.loader import write_model_folder
    import plain_llama as plain

    raw = {"architectures": ["ToyDecayForCausalLM"], "hidden_size": HIDDEN, "vocab_size": VOCAB,
           "num_hidden_layers": LAYERS, "eps": 1e-5, "decay": DECAY}
    arch = architecture_of(raw)
    specs = DecoderModel(arch.make_plan(raw), torch.float32, torch.device("cpu")).weight_specs()
    folder = write_model_folder(tmp_path / "toy", raw, specs, seed=11, std=0.15, norm_jitter=0.1, dtype=torch.float32)
    engine = Engine.from_pretrained(folder, dtype="float32", block_size=4, num_blocks=40, max_batch_size=3)
    layout = engine.model.cache_layout
    assert [s.name for s in layout.states] == ["toy_state@0", "toy_state@2"] and len(layout.groups) == 1
    assert layout.placement == [None, (0, 0), None]

    weights = plain.read_weights(folder)
    seqs = {"x": torch.randint(0, VOCAB, (23,), generator=torch.Generator().manual_seed(1)).tolist(),
            "y": torch.randint(0, VOCAB, (11,), generator=torch.Generator().manual_seed(2)).tolist()}
    want = {k: plain_toy(weights, raw, v) for k, v in seqs.items()}
    runner = engine.runner
    runner.admit("x"), runner.admit("y")
    got = {"x": [], "y": []}
    fed = {"x": 0, "y": 0}
    plan = [{"x": 5}, {"x": 2, "y": 4}, {"x": 1, "y": 1}, {"y": 6}, {"x": 15}]
    for step in plan:
        entries = [StepEntry(k, tokens=seqs[k][fed[k]: fed[k] + n], want=list(range(n))) for k, n in step.items()]
        logits = runner.step(entries).cpu()
        row = 0
        for k, n in step.items():
            got[k].append(logits[row: row + n])
            row += n
            fed[k] += n
    for k in seqs:
        torch.testing.assert_close(torch.cat(got[k]), want[k], atol=2e-4, rtol=2e-4)
    # a released slot starts from zero for the next request
    runner.release("x")
    runner.admit("z")
    again = runner.step([StepEntry("z", tokens=seqs["x"], want=[22])]).cpu()
    torch.testing.assert_close(again[0], want["x"][22], atol=2e-4, rtol=2e-4)


def test_windowed_attention_layers_release_pages_behind_the_window(tmp_path):
    """An architecture registered here whose layers alternate full and windowed attention: two cache
    groups with pages of their own; the windowed group gives pages back while the request runs (they are
    poisoned with NaN when freed), and the logits still equal a plain windowed computation."""
    from edgerag_b200 import Engine
    from edgerag_b200.config import register_architecture
    from edgerag_b200.config.registry import architecture_of
    from edgerag_b200.engine.step import StepEntry
    from edgerag_b200.models.decoder import DecoderModel
    from edgerag_b200.parts.base import LayerCall, LayerSpec, ModelPlan, PartSpec
    from edgerag_b200.weights.loader import write_model_folder
    import plain_llama as plain

    window, h, nq, nkv, d, inter, vocab, layers = 21, 40, 4, 2, 16, 56, 61, 4

    def make_plan(raw):
        norm = lambda p: PartSpec("rmsnorm", {"size": h, "eps": 1e-5}, p)   # noqa: E731
        specs = []
        for i in range(layers):
            mixer = PartSpec("attention", {"hidden": h, "n_q_heads": nq, "n_kv_heads": nkv, "head_dim": d,
                                           "window": window if i % 2 else 0,
                                           "position": PartSpec("rope_halves", {"head_dim": d, "theta": 500.0})}, "self_attn.")
            specs.append(LayerSpec(f"layers.{i}.", PartSpec("prenorm"), norm("ln1."), mixer, norm("ln2."),
                                   PartSpec("swiglu", {"hidden": h, "intermediate": inter}, "mlp.")))
        return ModelPlan(h, vocab, PartSpec("table", {"vocab": vocab, "hidden": h}, "embed_tokens."), specs,
                         [LayerCall(i, i) for i in range(layers)], norm("norm."),
                         PartSpec("linear", {"vocab": vocab, "hidden": h, "tied_to": None}, "lm_head."))

    register_architecture("ToyWindowForCausalLM", lambda raw, where: raw, make_plan)
    raw = {"architectures": ["ToyWindowForCausalLM"]}
    arch = architecture_of(raw)
    specs = DecoderModel(arch.make_plan(raw), torch.float32, torch.device("cpu")).weight_specs()
    folder = write_model_folder(tmp_path / "win", raw, specs, seed=5, std=0.2, norm_jitter=0.1, dtype=torch.float32)
    engine = Engine.from_pretrained(folder, dtype="float32", block_size=4, num_blocks=30, max_batch_size=2,
                                    poison_freed_pages=True)
    layout = engine.model.cache_layout
    assert [(g.n_layers, g.window) for g in layout.groups] == [(2, 0), (2, window)]
    assert layout.placement == [(0, 0), (1, 0), (0, 1), (1, 1)]

    w = plain.read_weights(folder)
    seq = torch.randint(0, vocab, (90,), generator=torch.Generator().manual_seed(3)).tolist()
    cfg = {"head_dim": d, "n_q": nq, "n_kv": nkv, "theta": 500.0}
    x = w["model.embed_tokens.weight"][torch.tensor(seq)]
    for i in range(layers):
        p = f"model.layers.{i}."
        a = p + "self_attn."
        x = x + plain.attention(plain.rms_norm(x, w[p + "ln1.weight"], 1e-5), torch.arange(len(seq)), w[a + "q_proj.weight"],
                                w[a + "k_proj.weight"], w[a + "v_proj.weight"], w[a + "o_proj.weight"], cfg,
                                window=window if i % 2 else None)
        m = p + "mlp."
        x = x + plain.swiglu(plain.rms_norm(x, w[p + "ln2.weight"], 1e-5), w[m + "gate_proj.weight"],
                             w[m + "up_proj.weight"], w[m + "down_proj.weight"])
    want = plain.rms_norm(x, w["model.norm.weight"], 1e-5) @ w["lm_head.weight"].T

    runner = engine.runner
    runner.admit("w")
    got, fed = [], 0
    for n in (30, 7, 1, 1, 1, 19, 1, 1, 2, 27):          # portions longer than the window, and single tokens
        got.append(runner.step([StepEntry("w", tokens=seq[fed: fed + n], want=list(range(n)))]).cpu().clone())
        fed += n
        engine.cache.check_invariants()
    assert fed == len(seq)
    torch.testing.assert_close(torch.cat(got), want, atol=2e-4, rtol=2e-4)
    held = engine.cache.held_pages("w")
    assert held[0] == 23 and held[1] <= (window + 3) // 4 + 1      # the windowed group kept only what is visible
    runner.release("w")
    assert engine.cache.free_pages() == [30, 30]


def test_toy_routed_feed_forward_and_another_position_encoding(tmp_path):
    """Two more parts defined here and registered from outside: a feed-forward that routes every token to
    two of five small experts (router logits and gates in float32), and a position encoding that turns
    neighbouring pairs of a head instead of its halves.  A plan mixes them with the framework's own parts
    layer by layer (dense and routed feed-forwards, both encodings in one model); the model is built,
    loaded and stepped in portions beside another request, in both element types, and its logits equal a
    whole-sequence computation written out below.  Neither part is a model of anyone's."""
    from edgerag_b200 import Engine
    from edgerag_b200.config import register_architecture
    from edgerag_b200.config.registry import architecture_of
    from edgerag_b200.engine.step import StepEntry
    from edgerag_b200.models.decoder import DecoderModel
    from edgerag_b200.ops import kernels
    from edgerag_b200.parts.base import (FeedForward, LayerCall, LayerSpec, ModelPlan, PartSpec, PositionEncoding, WeightSpec,
                                         register_part)
    from edgerag_b200.weights.loader import write_model_folder
    import plain_llama as plain

    h, nq, nkv, d, inter, vocab, layers = 40, 4, 2, 16, 56, 83, 3
    experts, top, e_inter, theta = 5, 2, 24, 300.0

    @register_part("ffn", "toy_routed")
    class ToyRoutedFeedForward(FeedForward):
        """y = sum over a token's two best experts of gate * down_e(relu(up_e(x))); gates: softmax over the two router logits."""

        def __init__(self, hidden, experts, top, intermediate, dtype, device):
            self.hidden, self.experts, self.top, self.intermediate = hidden, experts, top, intermediate
            self.dtype, self.device = dtype, device

        def weight_specs(self):
            specs = [WeightSpec("router.weight", (self.experts, self.hidden), kind="keep")]
            for e in range(self.experts):
                specs += [WeightSpec(f"experts.{e}.up.weight", (self.intermediate, self.hidden)),
                          WeightSpec(f"experts.{e}.down.weight", (self.hidden, self.intermediate))]
            return specs

        def load_weights(self, tensors):
            self.router = tensors["router.weight"].to(device=self.device, dtype=torch.float32)
            self.up = [tensors[f"experts.{e}.up.weight"].to(device=self.device, dtype=self.dtype) for e in range(self.experts)]
            self.down = [tensors[f"experts.{e}.down.weight"].to(device=self.device, dtype=self.dtype) for e in range(self.experts)]

        def forward(self, x, ctx):
            logits = x.float() @ self.router.T                                    # float32 router
            best, which = torch.topk(logits, self.top, dim=-1)
            gates = torch.softmax(best, dim=-1)
            y = torch.zeros((x.shape[0], self.hidden), dtype=torch.float32, device=x.device)
            for e in range(self.experts):
                weight = (gates * (which == e)).sum(dim=-1, keepdim=True)         # 0 for tokens that did not choose e
                mid = torch.empty((x.shape[0], self.intermediate), dtype=self.dtype, device=x.device)
                kernels.linear(x, self.up[e], mid)
                out = torch.empty((x.shape[0], self.hidden), dtype=self.dtype, device=x.device)
                kernels.linear(torch.relu(mid), self.down[e], out)
                y += weight * out.float()
            return y.to(self.dtype)

    @register_part("position", "toy_pairs")
    class ToyPairRotary(PositionEncoding):
        """Turns the pairs (x[2i], x[2i + 1]) of every q and k head by position * theta^(-2i / D), then writes k and v to the cache."""

        def __init__(self, head_dim, theta, dtype, device):
            self.inv_freq = (1.0 / theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim)).to(device)

        def apply_and_store(self, qkv, ctx, n_q_heads, n_kv_heads, head_dim, pages, slots):
            n = qkv.shape[0]
            angle = ctx.positions[:n].float()[:, None] * self.inv_freq[None]      # [n, D / 2]
            cos, sin = angle.cos()[:, None, :], angle.sin()[:, None, :]
            turned = qkv[:, : (n_q_heads + n_kv_heads) * head_dim].float().view(n, n_q_heads + n_kv_heads, head_dim // 2, 2)
            a, b = turned[..., 0], turned[..., 1]
            both = torch.stack((a * cos - b * sin, a * sin + b * cos), dim=-1).reshape(n, -1)
            qkv[:, : both.shape[1]] = both.to(qkv.dtype)
            if pages is not None:                                                 # rot_dim 0: the plain cache write
                kernels.rope_cache_write(qkv, ctx.positions, None, n_q_heads, n_kv_heads, head_dim, 0, slots=slots,
                                         k_pages=pages[0], v_pages=pages[1], page_size=ctx.page_size)

    def make_plan(raw):
        norm = lambda p: PartSpec("rmsnorm", {"size": h, "eps": 1e-5}, p)   # noqa: E731
        dense = PartSpec("swiglu", {"hidden": h, "intermediate": inter}, "mlp.")
        routed = PartSpec("toy_routed", {"hidden": h, "experts": experts, "top": top, "intermediate": e_inter}, "moe.")
        pairs = PartSpec("toy_pairs", {"head_dim": d, "theta": theta})
        halves = PartSpec("rope_halves", {"head_dim": d, "theta": theta})
        specs = []
        for i, (position, ffn) in enumerate([(pairs, dense), (halves, routed), (pairs, routed)]):
            mixer = PartSpec("attention", {"hidden": h, "n_q_heads": nq, "n_kv_heads": nkv, "head_dim": d, "position": position}, "self_attn.")
            specs.append(LayerSpec(f"layers.{i}.", PartSpec("prenorm"), norm("ln1."), mixer, norm("ln2."), ffn))
        return ModelPlan(h, vocab, PartSpec("table", {"vocab": vocab, "hidden": h}, "embed_tokens."), specs,
                         [LayerCall(i, i) for i in range(layers)], norm("norm."),
                         PartSpec("linear", {"vocab": vocab, "hidden": h, "tied_to": None}, "lm_head."))

    register_architecture("ToyRoutedForCausalLM", lambda raw, where: raw, make_plan)
    raw = {"architectures": ["ToyRoutedForCausalLM"]}
    specs = DecoderModel(architecture_of(raw).make_plan(raw), torch.float32, torch.device("cpu")).weight_specs()
    folder = write_model_folder(tmp_path / "routed", raw, specs, seed=9, std=0.2, norm_jitter=0.1, dtype=torch.float32)
    w = plain.read_weights(folder)

    def attention_with(turn, x, a):
        n = x.shape[0]
        q = (x @ w[a + "q_proj.weight"].T).view(n, nq, d).transpose(0, 1)
        k = (x @ w[a + "k_proj.weight"].T).view(n, nkv, d).transpose(0, 1)
        v = (x @ w[a + "v_proj.weight"].T).view(n, nkv, d).transpose(0, 1)
        return plain.attention_core(turn(q), turn(k), v, d ** -0.5) @ w[a + "o_proj.weight"].T

    def whole(seq):
        """The model on a whole sequence, float32, no cache: one expression per part."""
        n = len(seq)
        pos = torch.arange(n, dtype=torch.float32)
        angle = pos[:, None] / theta ** (torch.arange(0, d, 2, dtype=torch.float32) / d)[None]      # [n, D / 2]

        def pairs(t):       # [heads, n, D]
            a, b = t[..., 0::2], t[..., 1::2]
            return torch.stack((a * angle.cos() - b * angle.sin(), a * angle.sin() + b * angle.cos()), dim=-1).reshape(t.shape)

        cos, sin = plain.rope_tables(torch.arange(n), d, theta)
        halves = lambda t: plain.apply_rope(t, cos, sin)   # noqa: E731
        x = w["model.embed_tokens.weight"][torch.tensor(seq)]
        for i, (turn, routed) in enumerate([(pairs, False), (halves, True), (pairs, True)]):
            p = f"model.layers.{i}."
            x = x + attention_with(turn, plain.rms_norm(x, w[p + "ln1.weight"], 1e-5), p + "self_attn.")
            y = plain.rms_norm(x, w[p + "ln2.weight"], 1e-5)
            if not routed:
                m = p + "mlp."
                x = x + plain.swiglu(y, w[m + "gate_proj.weight"], w[m + "up_proj.weight"], w[m + "down_proj.weight"])
                continue
            best, which = torch.topk(y @ w[p + "moe.router.weight"].T, top, dim=-1)
            gates = torch.softmax(best, dim=-1)
            out = torch.zeros_like(x)
            for t in range(n):
                for g, e in zip(gates[t], which[t]):
                    m = f"{p}moe.experts.{int(e)}."
                    out[t] += g * (torch.relu(y[t] @ w[m + "up.weight"].T) @ w[m + "down.weight"].T)
            x = x + out
        return plain.rms_norm(x, w["model.norm.weight"], 1e-5) @ w["lm_head.weight"].T

    seqs = {"x": torch.randint(0, vocab, (37,), generator=torch.Generator().manual_seed(1)).tolist(),
            "y": torch.randint(0, vocab, (19,), generator=torch.Generator().manual_seed(2)).tolist()}
    want = {k: whole(v) for k, v in seqs.items()}
    assert len({int(e) for e in torch.topk(plain.rms_norm(w["model.embed_tokens.weight"], w["model.layers.1.ln2.weight"], 1e-5)
                                          @ w["model.layers.1.moe.router.weight"].T, top, dim=-1).indices.flatten()}) >= 4
    plan = [{"x": 9}, {"x": 2, "y": 6}, {"x": 1, "y": 1}, {"y": 12}, {"x": 25}]
    for dtype in ("float32", "bfloat16"):
        engine = Engine.from_pretrained(folder, dtype=dtype, block_size=4, num_blocks=40, max_batch_size=3)
        assert not engine.runner.graphs_enabled          # parts that do not declare themselves safe are never captured
        runner = engine.runner
        runner.admit("x"), runner.admit("y")
        got, fed = {"x": [], "y": []}, {"x": 0, "y": 0}
        for step in plan:
            entries = [StepEntry(k, tokens=seqs[k][fed[k]: fed[k] + n], want=list(range(n))) for k, n in step.items()]
            logits = runner.step(entries).cpu()
            row = 0
            for k, n in step.items():
                got[k].append(logits[row: row + n].clone())
                row += n
                fed[k] += n
        for k in seqs:
            out = torch.cat(got[k])
            if dtype == "float32":
                torch.testing.assert_close(out, want[k], atol=2e-4, rtol=2e-4)
            else:
                scale = float(want[k].abs().max())
                diff = (out - want[k]).abs()
                # a token whose two best router logits lie close may go to another expert in bfloat16: judge the rest
                assert float(diff.mean()) <= 0.01 * scale and float((diff.max(dim=1).values <= 0.03 * scale).float().mean()) >= 0.8


def test_toy_feed_forward_that_hands_over_partial_sums(tmp_path):
    """A feed-forward defined here whose last product leaves float32 partial sums over slices of k
    (``kernels.linear_parts``) instead of finished rows: the norm that follows (the next layer's, or the final
    one) adds them, so nothing outside the part changes.  Stepped in portions of 1 to 40 rows beside another
    request, in bfloat16 (partial sums) and in float32 (finished rows), against a whole-sequence computation."""
    from edgerag_b200 import Engine
    from edgerag_b200.config import register_architecture
    from edgerag_b200.config.registry import architecture_of
    from edgerag_b200.engine.step import StepEntry
    from edgerag_b200.models.decoder import DecoderModel
    from edgerag_b200.ops import kernels
    from edgerag_b200.parts.base import FeedForward, LayerCall, LayerSpec, ModelPlan, PartSpec, WeightSpec, register_part
    from edgerag_b200.weights.loader import write_model_folder
    import helpers
    import plain_llama as plain

    h, nq, nkv, d, inter, vocab, layers, theta = 48, 3, 1, 16, 200, 91, 2, 500.0
    handed_over = []

    @register_part("ffn", "toy_parts")
    class ToyPartsFeedForward(FeedForward):
        """y = down(relu(up(x))); up to 64 bfloat16 rows the down product is handed over as partial sums."""

        def __init__(self, hidden, intermediate, dtype, device):
            self.hidden, self.intermediate, self.dtype, self.device = hidden, intermediate, dtype, device

        def weight_specs(self):
            return [WeightSpec("up.weight", (self.intermediate, self.hidden)), WeightSpec("down.weight", (self.hidden, self.intermediate))]

        def load_weights(self, tensors):
            self.up = tensors["up.weight"].to(device=self.device, dtype=self.dtype).contiguous()
            self.down = tensors["down.weight"].to(device=self.device, dtype=self.dtype).contiguous()

        def forward(self, x, ctx):
            n = x.shape[0]
            mid = torch.empty((n, self.intermediate), dtype=self.dtype, device=x.device)
            kernels.linear(x, self.up, mid)
            mid = torch.relu(mid)
            if self.dtype == torch.bfloat16 and n <= kernels.TC_MAX_ROWS:
                parts = torch.empty((kernels.linear_parts_slices(self.down), n, self.hidden), dtype=torch.float32, device=x.device)
                kernels.linear_parts(mid, self.down, parts)
                handed_over.append(parts.shape[0])
                return parts
            y = torch.empty((n, self.hidden), dtype=self.dtype, device=x.device)
            kernels.linear(mid, self.down, y)
            return y

    def make_plan(raw):
        norm = lambda p: PartSpec("rmsnorm", {"size": h, "eps": 1e-5}, p)   # noqa: E731
        rope = PartSpec("rope_halves", {"head_dim": d, "theta": theta})
        specs = []
        for i in range(layers):
            mixer = PartSpec("attention", {"hidden": h, "n_q_heads": nq, "n_kv_heads": nkv, "head_dim": d, "position": rope}, "self_attn.")
            ffn = PartSpec("toy_parts", {"hidden": h, "intermediate": inter}, "ff.")
            specs.append(LayerSpec(f"layers.{i}.", PartSpec("prenorm"), norm("ln1."), mixer, norm("ln2."), ffn))
        return ModelPlan(h, vocab, PartSpec("table", {"vocab": vocab, "hidden": h}, "embed_tokens."), specs,
                         [LayerCall(i, i) for i in range(layers)], norm("norm."),
                         PartSpec("linear", {"vocab": vocab, "hidden": h, "tied_to": None}, "lm_head."))

    register_architecture("ToyPartsForCausalLM", lambda raw, where: raw, make_plan)
    raw = {"architectures": ["ToyPartsForCausalLM"]}
    specs = DecoderModel(architecture_of(raw).make_plan(raw), torch.float32, torch.device("cpu")).weight_specs()
    folder = write_model_folder(tmp_path / "parts", raw, specs, seed=13, std=0.2, norm_jitter=0.1, dtype=torch.float32)
    w = plain.read_weights(folder)
    cfg = {"n_q": nq, "n_kv": nkv, "head_dim": d, "theta": theta}

    def whole(seq):
        x = w["model.embed_tokens.weight"][torch.tensor(seq)]
        pos = torch.arange(len(seq))
        for i in range(layers):
            p = f"model.layers.{i}."
            a = p + "self_attn."
            x = x + plain.attention(plain.rms_norm(x, w[p + "ln1.weight"], 1e-5), pos, w[a + "q_proj.weight"], w[a + "k_proj.weight"],
                                    w[a + "v_proj.weight"], w[a + "o_proj.weight"], cfg)
            y = plain.rms_norm(x, w[p + "ln2.weight"], 1e-5)
            x = x + torch.relu(y @ w[p + "ff.up.weight"].T) @ w[p + "ff.down.weight"].T
        return plain.rms_norm(x, w["model.norm.weight"], 1e-5) @ w["lm_head.weight"].T

    seqs = {"x": torch.randint(0, vocab, (70,), generator=torch.Generator().manual_seed(3)).tolist(),
            "y": torch.randint(0, vocab, (31,), generator=torch.Generator().manual_seed(4)).tolist()}
    want = {k: whole(v) for k, v in seqs.items()}
    plan = [{"x": 9}, {"x": 2, "y": 17}, {"x": 1, "y": 1}, {"y": 13}, {"x": 40}, {"x": 18}]
    for dtype in ("float32", "bfloat16"):
        engine = Engine.from_pretrained(folder, dtype=dtype, block_size=4, num_blocks=60, max_batch_size=3)
        runner = engine.runner
        runner.admit("x"), runner.admit("y")
        got, fed = {"x": [], "y": []}, {"x": 0, "y": 0}
        for step in plan:
            entries = [StepEntry(k, tokens=seqs[k][fed[k]: fed[k] + n], want=list(range(n))) for k, n in step.items()]
            logits = runner.step(entries).cpu()
            row = 0
            for k, n in step.items():
                got[k].append(logits[row: row + n].clone())
                row += n
                fed[k] += n
        for k in seqs:
            out = torch.cat(got[k])
            if dtype == "float32":
                torch.testing.assert_close(out, want[k], atol=2e-4, rtol=2e-4)
            else:
                scale = float(want[k].abs().max())
                diff = (out - want[k]).abs()
                assert float(diff.max()) <= helpers.BF16_FRACTION * scale and float(diff.mean()) <= helpers.BF16_MEAN_FRACTION * scale
    assert handed_over and min(handed_over) >= 2       # k = 200 is cut into more than one slice
