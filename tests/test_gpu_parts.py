"""Each part alone against the plain implementation's function for it, and the
generality of the assembly: a toy mixer with state of its own, defined here,
is registered, built into a model beside attention layers, loaded from a
folder the random-weights mode wrote, and stepped in several cuttings, without
a change to the library's files. The toy model's schedule also names a layer
twice and lets its second run read the first run's cache."""
import json
import math
import os

import numpy as np
import pytest
import torch

import plain_llama as plain
import tiny

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def make_ctx(cache, slots, token_lists, vocab=1000, want=None):
    from foundry_b200.engine import SequenceStep, build_context
    steps = [SequenceStep(s, t, list(range(len(t))) if want is None else want)
             for s, t in zip(slots, token_lists)]
    return build_context(cache, steps, vocab, DEV)


def tol(dtype):
    return dict(atol=3e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=4e-2, rtol=2e-2)


def assert_close(got, want, dtype, scale=1.0):
    t = tol(dtype)
    got, want = got.double().cpu(), want.double().cpu()
    err = (got - want).abs()
    bound = t["atol"] * scale + t["rtol"] * want.abs()
    frac = float((err <= bound).double().mean())
    assert frac >= (1.0 if dtype == torch.float32 else 0.999), \
        f"{frac:.5f} close, max err {float(err.max()):.3e}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rms_norm_part(dtype):
    from foundry_b200.parts import RMSNorm
    part = RMSNorm(96, 1e-6, dtype=dtype, device=DEV)
    w = (1 + 0.1 * torch.randn(96)).to(dtype)
    part.load("n", lambda name: w.to(DEV))
    resid = torch.randn(7, 96, device=DEV)
    delta = torch.randn(7, 96, device=DEV).to(dtype)
    r0 = resid.clone()
    out = part.add_norm(resid, delta)
    want = plain.rms_norm(r0.double().cpu() + delta.double().cpu(), w.double(), 1e-6)
    assert out.dtype == dtype
    assert_close(out, want, dtype)
    listed = part.expected_tensors("x.norm")
    assert list(listed) == ["x.norm.weight"] and tuple(listed["x.norm.weight"].shape) == (96,)
    assert not listed["x.norm.weight"].integer


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu_part(dtype):
    from foundry_b200.parts import SwiGLU
    H, I, T = 96, 176, 9
    part = SwiGLU(H, I, dtype=dtype, device=DEV)
    w = {f"m.{n}.weight": (0.1 * torch.randn(*s)).to(dtype)
         for n, s in (("gate_proj", (I, H)), ("up_proj", (I, H)), ("down_proj", (H, I)))}
    assert {k: v.shape for k, v in part.expected_tensors("m").items()} == \
        {k: tuple(v.shape) for k, v in w.items()}
    part.load("m", lambda name: w[name].to(DEV))
    x = torch.randn(T, H).to(dtype)
    got = part.forward(None, x.to(DEV))
    want = plain.mlp(x.double(), {k: v.double() for k, v in w.items()}, "m")
    assert_close(got, want, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", ["tiny_a", "tiny_b"])
def test_attention_part_alone_in_two_cuttings(name, dtype):
    """The mixer with a cache of its own: whole sequences of unequal lengths in
    one step, and the same split into a prompt part and single tokens."""
    from foundry_b200.cache import SequenceCache
    from foundry_b200.config import LlamaConfig
    from foundry_b200.models.llama import build_llama_spec
    from foundry_b200.parts import MIXERS
    cfg = tiny.CONFIGS[name]
    spec = build_llama_spec(LlamaConfig.parse(cfg))
    part = MIXERS.build(spec.layers[0].mixer, dtype=dtype, device=DEV)
    H = cfg["hidden_size"]
    torch.manual_seed(1)
    w = {k: (0.15 * torch.randn(*e.shape)).to(dtype) for k, e in part.expected_tensors("a").items()}
    part.load("a", lambda n: w[n].to(DEV))
    cache = SequenceCache({0: part.cache_request()}, 1024, 4, dtype, DEV)
    lens = [70, 3, 33]
    xs = [torch.randn(n, H).to(dtype) for n in lens]
    wd = {k: v.double() for k, v in w.items()}
    want = [plain.attention(x.double(), wd, "a", cfg, list(range(len(x)))) for x in xs]

    slots = [cache.open_sequence() for _ in lens]
    ctx = make_ctx(cache, slots, [[0] * n for n in lens])
    got = part.forward(ctx, torch.cat(xs).to(DEV), cache.view(0, True))
    assert_close(got, torch.cat(want), dtype, scale=float(torch.cat(want).abs().max()))
    for s in slots:
        cache.close_sequence(s)

    slots = [cache.open_sequence() for _ in lens]
    head = [max(1, n - 2) for n in lens]
    ctx = make_ctx(cache, slots, [[0] * h for h in head])
    outs = [part.forward(ctx, torch.cat([x[:h] for x, h in zip(xs, head)]).to(DEV), cache.view(0, True))]
    pieces = {i: [o] for i, o in enumerate(torch.split(outs[0], head))}
    for step in range(2):
        live = [i for i, n in enumerate(lens) if head[i] + step < n]
        ctx = make_ctx(cache, [slots[i] for i in live], [[0]] * len(live))
        o = part.forward(ctx, torch.cat([xs[i][head[i] + step:head[i] + step + 1] for i in live]).to(DEV),
                         cache.view(0, True))
        for j, i in enumerate(live):
            pieces[i].append(o[j:j + 1])
    got = torch.cat([torch.cat(pieces[i]) for i in range(len(lens))])
    assert_close(got, torch.cat(want), dtype, scale=float(torch.cat(want).abs().max()))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", ["tiny_a", "tiny_b"])
def test_block_part_alone(name, dtype):
    """The arrangement of a layer's parts, built from its description alone and
    run on residual rows of its own: x + mixer(norm(x)), then + feed-forward(norm(.)),
    against the plain decoder layer; whole sequences, then the same with the last
    tokens one by one (where the norms ride on the projections)."""
    from foundry_b200.cache import SequenceCache
    from foundry_b200.config import LlamaConfig
    from foundry_b200.models.llama import build_llama_spec
    from foundry_b200.parts import BLOCKS
    cfg = tiny.CONFIGS[name]
    spec = build_llama_spec(LlamaConfig.parse(cfg))
    layer = spec.layers[1]
    block = BLOCKS.build(layer.block, layer=layer, dtype=dtype, device=DEV)
    torch.manual_seed(3)
    w = {k: ((1.0 + 0.1 * torch.randn(*e.shape)) if len(e.shape) == 1 else 0.1 * torch.randn(*e.shape)).to(dtype)
         for k, e in block.expected_tensors().items()}
    assert all(k.startswith("model.layers.1.") for k in w)
    block.load(block.prefix, lambda n: w[n].to(DEV))
    cache = SequenceCache({0: block.cache_request()}, 512, 4, dtype, DEV)
    H = cfg["hidden_size"]
    lens = [37, 5, 66]
    xs = [torch.randn(n, H) for n in lens]
    wd = {k: v.double() for k, v in w.items()}
    want = [plain.decoder_layer(x.double(), wd, 1, cfg, list(range(len(x)))) for x in xs]

    def run(ctx, rows):
        resid = torch.cat(rows).to(DEV).float().contiguous()
        delta = block.forward(ctx, resid, None, cache.view(0, True))
        from foundry_b200.kernels import ops
        if isinstance(delta, ops.Planes):
            delta = delta.sum(dtype)
        return resid.double().cpu() + delta.double().cpu()  # the block returns its last part un-added

    slots = [cache.open_sequence() for _ in lens]
    head = [n - 3 for n in lens]
    got = [list(torch.split(run(make_ctx(cache, slots, [[0] * h for h in head]),
                                [x[:h] for x, h in zip(xs, head)]), head))]
    for step in range(3):
        out = run(make_ctx(cache, slots, [[0]] * len(lens)),
                  [x[h + step:h + step + 1] for x, h in zip(xs, head)])
        got.append(list(torch.split(out, [1] * len(lens))))
    for i in range(len(lens)):
        whole = torch.cat([piece[i] for piece in got])
        assert_close(whole, want[i], dtype, scale=float(want[i].abs().max()))


def test_position_encoding_parts_follow_the_reference_bands():
    """llama3 scaling at D = 128, theta = 5e5, factor 32: the three frequencies
    the reference pins (j = 0 unscaled, j = 32 blended, j = 63 divided;
    src/models/llama/rotary_emb.rs:203-239) against a float64 restatement."""
    from foundry_b200.parts import llama3_inv_freq, plain_inv_freq
    got = llama3_inv_freq(128, 500000.0, 32.0, 1.0, 4.0, 8192)
    for j in (0, 32, 63):
        f = 500000.0 ** (-2.0 * j / 128)
        wl = 2 * math.pi / f
        if wl < 8192 / 4:
            want = f
        elif wl > 8192 / 1:
            want = f / 32
        else:
            s = (8192 / wl - 1.0) / (4.0 - 1.0)
            want = (1 - s) * f / 32 + s * f
        assert abs(got[j] - want) <= 1e-5 * want, j
    assert got.dtype == np.float32 and got.shape == (64,)
    plain64 = plain_inv_freq(64, 100000.0)  # rotary_emb.rs:241-259
    for j in (0, 16, 31):
        assert abs(plain64[j] - 100000.0 ** (-2.0 * j / 64)) <= 1e-5 * 100000.0 ** (-2.0 * j / 64)
    # equal to the plain implementation's own restatement, element for element
    for name in ("tiny_a", "tiny_b"):
        cfg = tiny.CONFIGS[name]
        rs = cfg["rope_scaling"]
        mine = plain_inv_freq(cfg["head_dim"], cfg["rope_theta"]) if rs is None else \
            llama3_inv_freq(cfg["head_dim"], cfg["rope_theta"], rs["factor"], rs["low_freq_factor"],
                            rs["high_freq_factor"], rs["original_max_position_embeddings"])
        assert np.array_equal(mine, plain.inv_freq(cfg))


# --------------------------------------------------------------- the toy model
def register_toy():
    """A mixer with a fixed-size state per sequence: y_t = W * mean(x_0..x_t).
    The state row of a sequence holds the running sum. Everything it needs
    comes through the part interfaces and the step context."""
    from foundry_b200.cache import StateRequest
    from foundry_b200.config import (Architecture, LayerSpec, LlamaConfig, ModelSpec, PartSpec,
                                     ScheduleEntry, register_architecture)
    from foundry_b200.parts import Linear, Part, register_mixer

    class RunningMean(Part):
        def __init__(self, hidden_size, *, dtype, device):
            self.h, self.dtype = hidden_size, dtype
            self.proj = Linear(hidden_size, [("proj", hidden_size)], dtype=dtype, device=device)

        def expected_tensors(self, prefix):
            return self.proj.expected_tensors(prefix)

        def load(self, prefix, fetch):
            self.proj.load(prefix, fetch)

        def cache_request(self):
            return StateRequest((self.h,), torch.float32)

        def forward(self, ctx, x, state):
            # Reads the step on the host in every kind of step, single-token steps
            # included: the part does not set `replay_safe`, so the engine must
            # launch its steps plainly and hand it the host copies (a captured
            # step would replay the first step's slots and lengths for ever).
            assert ctx.slots_host is not None and ctx.cu_tokens_host is not None
            xf = x.float()
            parts = []
            for i, slot in enumerate(ctx.slots_host):
                a, b = ctx.cu_tokens_host[i], ctx.cu_tokens_host[i + 1]
                total = state.rows[slot] + torch.cumsum(xf[a:b], 0)
                state.rows[slot] = total[-1]
                parts.append(total)
            mean = torch.cat(parts) / (ctx.positions.float() + 1.0).unsqueeze(1)
            return self.proj.forward(mean.to(self.dtype))

    register_mixer("toy_running_mean", RunningMean, replace=True)

    def build_spec(config):
        from foundry_b200.models.llama import HF_NAMES, build_llama_spec
        llama = build_llama_spec(config)
        attn_layer = llama.layers[0]
        toy_layer = LayerSpec(prefix="model.layers.1", block=attn_layer.block,
                              mixer=PartSpec("toy_running_mean", {"hidden_size": config.hidden_size}),
                              feed_forward=attn_layer.feed_forward, mixer_norm=attn_layer.mixer_norm,
                              feed_forward_norm=attn_layer.feed_forward_norm,
                              names={**HF_NAMES, "mixer": "toy"})
        spec = ModelSpec(
            architecture="ToyForCausalLM", hidden_size=llama.hidden_size,
            vocab_size=llama.vocab_size, max_positions=llama.max_positions,
            layers=(attn_layer, toy_layer),
            # layer 0 runs twice with the same weights; its second run reads the keys
            # and values its first run wrote
            schedule=(ScheduleEntry(0, 0), ScheduleEntry(1, 1), ScheduleEntry(0, 0, writes_cache=False)),
            final_norm=llama.final_norm, embedding_name=llama.embedding_name,
            final_norm_prefix=llama.final_norm_prefix, output_head_name=llama.output_head_name)
        spec.validate()
        return spec

    class ToyConfig(LlamaConfig):
        pass

    def parse(doc):
        return LlamaConfig.parse({**doc, "architectures": ["ToyForCausalLM"]})

    register_architecture(Architecture("ToyForCausalLM", "llama", parse, build_spec), replace=True)


def toy_plain_forward(cfg, w, tokens):
    """The toy model, whole sequence, float64."""
    ids = torch.as_tensor(tokens)
    x = w["model.embed_tokens.weight"][ids]
    eps = cfg["rms_norm_eps"]
    positions = list(range(len(tokens)))
    S, A = len(tokens), cfg["num_attention_heads"]
    K, D = cfg["num_key_value_heads"], cfg["head_dim"]
    cos, sin = plain.rotary_tables(cfg, positions)
    p0 = "model.layers.0"

    def attn(xin, kv=None):
        n = plain.rms_norm(xin, w[f"{p0}.input_layernorm.weight"], eps)
        q = plain.apply_rotary((n @ w[f"{p0}.self_attn.q_proj.weight"].T).reshape(S, A, D), cos, sin)
        if kv is None:
            k = plain.apply_rotary((n @ w[f"{p0}.self_attn.k_proj.weight"].T).reshape(S, K, D), cos, sin)
            v = (n @ w[f"{p0}.self_attn.v_proj.weight"].T).reshape(S, K, D)
        else:
            k, v = kv
        out = torch.empty(S, A, D, dtype=torch.float64)
        mask = torch.tril(torch.ones(S, S, dtype=torch.bool))
        for a in range(A):
            s = (q[:, a] @ k[:, a // (A // K)].T) / math.sqrt(D)
            s = s.masked_fill(~mask, float("-inf"))
            out[:, a] = torch.softmax(s, -1) @ v[:, a // (A // K)]
        return out.reshape(S, A * D) @ w[f"{p0}.self_attn.o_proj.weight"].T, (k, v)

    def layer0(xin, kv=None):
        a, kv = attn(xin, kv)
        h = xin + a
        return h + plain.mlp(plain.rms_norm(h, w[f"{p0}.post_attention_layernorm.weight"], eps), w,
                             f"{p0}.mlp"), kv

    x, kv = layer0(x)
    p1 = "model.layers.1"
    n = plain.rms_norm(x, w[f"{p1}.input_layernorm.weight"], eps)
    mean = torch.cumsum(n, 0) / torch.arange(1, S + 1, dtype=torch.float64).unsqueeze(1)
    h = x + mean @ w[f"{p1}.toy.proj.weight"].T
    x = h + plain.mlp(plain.rms_norm(h, w[f"{p1}.post_attention_layernorm.weight"], eps), w, f"{p1}.mlp")
    x, _ = layer0(x, kv)
    x = plain.rms_norm(x, w["model.norm.weight"], eps)
    head = w["lm_head.weight"] if "lm_head.weight" in w else w["model.embed_tokens.weight"]
    return x @ head.T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_toy_mixer_with_state_is_registered_built_and_stepped(tmp_path, dtype):
    import foundry_b200 as fb
    from foundry_b200.config import LlamaConfig, unregister_architecture
    from foundry_b200.engine import SequenceStep
    from foundry_b200.parts import MIXERS
    register_toy()
    try:
        cfg = {**tiny.CONFIGS["tiny_b"], "architectures": ["ToyForCausalLM"], "num_hidden_layers": 2}
        folder = fb.write_model_folder(str(tmp_path / "toy"), LlamaConfig.parse(cfg), 5, std=0.08)
        assert json.load(open(os.path.join(folder, "config.json")))["architectures"] == ["ToyForCausalLM"]
        pcfg, w = plain.read_model(folder)
        assert "model.layers.1.toy.proj.weight" in w and "model.layers.1.self_attn.q_proj.weight" not in w
        engine = fb.Engine.from_folder(folder, dtype=dtype, max_tokens=1024, max_slots=4)
        assert len(engine.cache.groups) == 1 and list(engine.cache.state) == [1]
        reqs = [tiny.random_tokens(300 + i, n, cfg["vocab_size"]) for i, n in enumerate((40, 5, 90, 67))]
        want = [toy_plain_forward(pcfg, w, r).numpy() for r in reqs]
        # whole
        for r, e in zip(reqs, want):
            s = engine.open_sequence()
            got = engine.step([SequenceStep(s, r, list(range(len(r))))]).cpu().numpy()
            engine.close_sequence(s)
            tiny.assert_logits_close(got, e, dtype, "toy whole")
        # batches of two (so slots and their state rows are used again), prompt then tokens
        for pair in ((0, 1), (2, 3), (1, 3)):
            slots = {i: engine.open_sequence() for i in pair}
            done = {i: max(1, len(reqs[i]) - 6) for i in pair}
            rows = {i: [] for i in pair}
            out = engine.step([SequenceStep(slots[i], reqs[i][:done[i]], list(range(done[i])))
                               for i in pair]).cpu().numpy()
            at = 0
            for i in pair:
                rows[i].append(out[at:at + done[i]])
                at += done[i]
            for _ in range(6):
                live = [i for i in pair if done[i] < len(reqs[i])]
                out = engine.step([SequenceStep(slots[i], [reqs[i][done[i]]], [0]) for i in live]).cpu().numpy()
                for j, i in enumerate(live):
                    rows[i].append(out[j:j + 1])
                    done[i] += 1
            for i in pair:
                engine.close_sequence(slots[i])
                tiny.assert_logits_close(np.concatenate(rows[i]), want[i], dtype, f"toy batched {pair}")
    finally:
        unregister_architecture("ToyForCausalLM")
        MIXERS.unregister("toy_running_mean")


@pytest.mark.parametrize("pairing", ["half", "interleaved"])
def test_a_toy_position_encoding_and_feed_forward_are_registered_and_run(tmp_path, pairing):
    """Two more parts defined here and plugged in by name: a position encoding
    that rotates only half of each head with linearly scaled frequencies (its
    pairs being elements i and i + width/2, or 2i and 2i + 1), and a
    feed-forward with a squared-ReLU and two token-routed experts (routing in
    32-bit). The attention part, the block and the engine are used unchanged."""
    import foundry_b200 as fb
    from foundry_b200.config import (Architecture, LlamaConfig, PartSpec, register_architecture,
                                     unregister_architecture)
    from foundry_b200.parts import (FEED_FORWARDS, POSITION_ENCODINGS, Linear, Part,
                                    register_feed_forward, register_position_encoding)
    from foundry_b200.engine import SequenceStep
    from dataclasses import replace

    class HalfRotary(Part):
        attention_factor = 1.0

        def __init__(self, head_dim, theta, scale, pairing, *, dtype=None, device=None):
            self.pairing = pairing
            self.rotary_dim = head_dim // 2
            inv = (1.0 / (theta ** (np.arange(0, self.rotary_dim, 2, dtype=np.float32) / self.rotary_dim))
                   / np.float32(scale)).astype(np.float32)
            self.inv_freq_host = inv
            self.inv_freq = torch.from_numpy(inv).to(device)

    class RoutedRelu2(Part):
        """y = sum over the top-1 expert e of softmax(router x)[e] * W2_e relu(W1_e x)^2."""

        def __init__(self, hidden_size, intermediate_size, experts, *, dtype, device):
            self.h, self.i, self.n, self.dtype = hidden_size, intermediate_size, experts, dtype
            self.router = Linear(hidden_size, [("router", experts)], dtype=dtype, device=device)
            self.up = [Linear(hidden_size, [(f"experts.{e}.up", intermediate_size)], dtype=dtype, device=device)
                       for e in range(experts)]
            self.down = [Linear(intermediate_size, [(f"experts.{e}.down", hidden_size)], dtype=dtype, device=device)
                         for e in range(experts)]

        def expected_tensors(self, prefix):
            out = dict(self.router.expected_tensors(prefix))
            for lin in self.up + self.down:
                out.update(lin.expected_tensors(prefix))
            return out

        def load(self, prefix, fetch):
            for lin in [self.router] + self.up + self.down:
                lin.load(prefix, fetch)

        def forward(self, ctx, x):
            gate = torch.softmax(self.router.forward(x, out_dtype=torch.float32), -1)  # 32-bit
            choice = gate.argmax(-1)
            y = torch.zeros(x.shape[0], self.h, dtype=torch.float32, device=x.device)
            for e in range(self.n):  # every expert on every token, masked: a toy, not a fast path
                hidden = torch.relu(self.up[e].forward(x).float()) ** 2
                out = self.down[e].forward(hidden.to(self.dtype)).float()
                y += out * (gate[:, e] * (choice == e)).unsqueeze(1)
            return y.to(self.dtype)

    register_position_encoding("toy_half_rotary", HalfRotary, replace=True)
    register_feed_forward("toy_routed_relu2", RoutedRelu2, replace=True)

    def build_spec(config, routed=True, name="Toy2ForCausalLM"):
        from foundry_b200.models.llama import build_llama_spec
        base = build_llama_spec(config)
        layers = []
        for layer in base.layers:
            mixer = PartSpec("gqa_attention", {**layer.mixer.params, "position_encoding": PartSpec(
                "toy_half_rotary", {"head_dim": config.head_dim, "theta": 10000.0, "scale": 2.0,
                                    "pairing": pairing})})
            ff = PartSpec("toy_routed_relu2", {"hidden_size": config.hidden_size,
                                               "intermediate_size": 48, "experts": 2})
            layers.append(replace(layer, mixer=mixer, feed_forward=ff if routed else layer.feed_forward))
        return replace(base, architecture=name, layers=tuple(layers))

    register_architecture(Architecture("Toy2ForCausalLM", "llama",
                                       lambda d: LlamaConfig.parse({**d, "architectures": ["Toy2ForCausalLM"]}),
                                       build_spec), replace=True)
    # the same position encoding with the ordinary feed-forward: for the 16-bit run,
    # in which a routed toy could send a token to the other expert on a near tie
    register_architecture(Architecture("Toy3ForCausalLM", "llama",
                                       lambda d: LlamaConfig.parse({**d, "architectures": ["Toy3ForCausalLM"]}),
                                       lambda c: build_spec(c, routed=False, name="Toy3ForCausalLM")),
                          replace=True)
    try:
        cfg_doc = {**tiny.CONFIGS["tiny_b"], "architectures": ["Toy2ForCausalLM"], "num_hidden_layers": 2}
        folder = fb.write_model_folder(str(tmp_path / "toy2"), LlamaConfig.parse(cfg_doc), 8, std=0.1)
        cfg, w = plain.read_model(folder)
        assert "model.layers.0.mlp.experts.1.down.weight" in w and "model.layers.0.mlp.router.weight" in w

        def plain_forward(tokens, w=w, routed=True):
            S, A, K, D = len(tokens), cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
            x = w["model.embed_tokens.weight"][torch.as_tensor(tokens)]
            rot = D // 2
            inv = (1.0 / (10000.0 ** (np.arange(0, rot, 2, dtype=np.float32) / rot)) / np.float32(2.0)).astype(np.float32)
            ang = (np.arange(S, dtype=np.float32)[:, None] * inv[None, :]).astype(np.float64)
            cos, sin = torch.from_numpy(np.cos(ang)), torch.from_numpy(np.sin(ang))

            def rope(t):  # [S, heads, D]: the pairs lie inside the first `rot` elements
                if pairing == "interleaved":  # (2i, 2i + 1)
                    a, b = t[..., 0:rot:2], t[..., 1:rot:2]
                    turned = torch.stack([a * cos[:, None] - b * sin[:, None],
                                          b * cos[:, None] + a * sin[:, None]], -1)
                    return torch.cat([turned.reshape(*t.shape[:-1], rot), t[..., rot:]], -1)
                a, b = t[..., :rot // 2], t[..., rot // 2:rot]  # (i, i + rot/2)
                return torch.cat([a * cos[:, None] - b * sin[:, None], b * cos[:, None] + a * sin[:, None],
                                  t[..., rot:]], -1)
            for i in range(2):
                p = f"model.layers.{i}"
                n = plain.rms_norm(x, w[f"{p}.input_layernorm.weight"], cfg["rms_norm_eps"])
                q = rope((n @ w[f"{p}.self_attn.q_proj.weight"].T).reshape(S, A, D))
                k = rope((n @ w[f"{p}.self_attn.k_proj.weight"].T).reshape(S, K, D))
                v = (n @ w[f"{p}.self_attn.v_proj.weight"].T).reshape(S, K, D)
                att = torch.empty(S, A, D, dtype=torch.float64)
                mask = torch.tril(torch.ones(S, S, dtype=torch.bool))
                for a_ in range(A):
                    s = (q[:, a_] @ k[:, a_ // (A // K)].T) / math.sqrt(D)
                    att[:, a_] = torch.softmax(s.masked_fill(~mask, float("-inf")), -1) @ v[:, a_ // (A // K)]
                h = x + att.reshape(S, A * D) @ w[f"{p}.self_attn.o_proj.weight"].T
                n = plain.rms_norm(h, w[f"{p}.post_attention_layernorm.weight"], cfg["rms_norm_eps"])
                if not routed:
                    x = h + plain.mlp(n, w, f"{p}.mlp")
                    continue
                gate = torch.softmax(n @ w[f"{p}.mlp.router.weight"].T, -1)
                choice = gate.argmax(-1)
                y = torch.zeros_like(h)
                for e in range(2):
                    hid = torch.relu(n @ w[f"{p}.mlp.experts.{e}.up.weight"].T) ** 2
                    y += (hid @ w[f"{p}.mlp.experts.{e}.down.weight"].T) * (gate[:, e] * (choice == e)).unsqueeze(1)
                x = h + y
            x = plain.rms_norm(x, w["model.norm.weight"], cfg["rms_norm_eps"])
            return (x @ w["lm_head.weight"].T).numpy()

        engine = fb.Engine.from_folder(folder, dtype="float32", max_tokens=512, max_slots=2)
        tokens = tiny.random_tokens(77, 50, cfg["vocab_size"])
        want = plain_forward(tokens)
        slot = engine.open_sequence()
        got = [engine.step([SequenceStep(slot, tokens[:45], list(range(45)))]).cpu().numpy()]
        for t in tokens[45:]:
            got.append(engine.step([SequenceStep(slot, [t], [0])]).cpu().numpy())
        engine.close_sequence(slot)
        got = np.concatenate(got)
        tiny.assert_logits_close(got, want, "float32", "toy position encoding and feed-forward")

        # the position encoding alone in both dtypes: in 16 bits single-token steps
        # rotate in the q/k/v product's epilogue, prompts in the rotary kernel
        doc3 = {**cfg_doc, "architectures": ["Toy3ForCausalLM"]}
        folder3 = fb.write_model_folder(str(tmp_path / "toy3"), LlamaConfig.parse(doc3), 9, std=0.1)
        _, w3 = plain.read_model(folder3)
        want = plain_forward(tokens, w3, routed=False)
        for dtype in ("float32", "bfloat16"):
            engine = fb.Engine.from_folder(folder3, dtype=dtype, max_tokens=512, max_slots=2)
            slot = engine.open_sequence()
            got = [engine.step([SequenceStep(slot, tokens[:30], list(range(30)))]).cpu().numpy()]
            for t in tokens[30:]:
                got.append(engine.step([SequenceStep(slot, [t], [0])]).cpu().numpy())
            engine.close_sequence(slot)
            tiny.assert_logits_close(np.concatenate(got), want, dtype, f"toy position encoding, {dtype}")
    finally:
        unregister_architecture("Toy2ForCausalLM")
        unregister_architecture("Toy3ForCausalLM")
        POSITION_ENCODINGS.unregister("toy_half_rotary")
        FEED_FORWARDS.unregister("toy_routed_relu2")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_windowed_layer_beside_a_full_one(tmp_path, dtype):
    """A toy architecture whose second layer attends to a window of 100 keys
    while its first sees all of them: two cache groups, the windowed one a ring
    of three pages. Prompts far longer than the ring (the engine feeds them in
    portions that leave every window intact), a prompt cut so that a portion
    ends exactly at the window's edge, and decoding past the ring's wrap, all
    against the plain model with the same window."""
    import foundry_b200 as fb
    from dataclasses import replace
    from foundry_b200.config import (Architecture, LlamaConfig, PartSpec, register_architecture,
                                     unregister_architecture)
    from foundry_b200.engine import SequenceStep
    W = 100

    def build_spec(config):
        from foundry_b200.models.llama import build_llama_spec
        base = build_llama_spec(config)
        layers = list(base.layers)
        layers[1] = replace(layers[1], mixer=PartSpec("gqa_attention",
                                                      {**layers[1].mixer.params, "window": W}))
        return replace(base, architecture="ToyWindowForCausalLM", layers=tuple(layers))

    register_architecture(Architecture(
        "ToyWindowForCausalLM", "llama",
        lambda d: LlamaConfig.parse({**d, "architectures": ["ToyWindowForCausalLM"]}), build_spec),
        replace=True)
    try:
        doc = {**tiny.CONFIGS["tiny_b"], "architectures": ["ToyWindowForCausalLM"],
               "num_hidden_layers": 2, "max_position_embeddings": 640}
        folder = fb.write_model_folder(str(tmp_path / "window"), LlamaConfig.parse(doc), 21, std=0.1)
        cfg, w = plain.read_model(folder)

        def plain_forward(tokens):
            x = w["model.embed_tokens.weight"][torch.as_tensor(tokens)]
            positions = list(range(len(tokens)))
            for i, window in enumerate((None, W)):
                p = f"model.layers.{i}"
                n = plain.rms_norm(x, w[f"{p}.input_layernorm.weight"], cfg["rms_norm_eps"])
                h = x + plain.attention(n, w, f"{p}.self_attn", cfg, positions, window=window)
                n = plain.rms_norm(h, w[f"{p}.post_attention_layernorm.weight"], cfg["rms_norm_eps"])
                x = h + plain.mlp(n, w, f"{p}.mlp")
            x = plain.rms_norm(x, w["model.norm.weight"], cfg["rms_norm_eps"])
            return (x @ w["lm_head.weight"].T).numpy()

        engine = fb.Engine.from_folder(folder, dtype=dtype, max_tokens=2048, max_slots=3)
        assert len(engine.cache.groups) == 2
        assert sorted(g.ring_pages for g in engine.cache.groups) == [0, 3]
        assert engine.cache.step_token_limit() == 3 * 64 - W + 1
        reqs = [tiny.random_tokens(400 + i, n, cfg["vocab_size"]) for i, n in enumerate((600, 93, 250))]
        want = [plain_forward(r) for r in reqs]
        # each whole in one call (600 tokens are seven portions of 93)
        for i, r in enumerate(reqs):
            s = engine.open_sequence()
            got = engine.step([SequenceStep(s, r, list(range(len(r))))]).cpu().numpy()
            engine.close_sequence(s)
            tiny.assert_logits_close(got, want[i], dtype, f"windowed, whole, request {i}")
        # all three in one batch: a prompt part, a second part, then single tokens to the end
        slots = [engine.open_sequence() for _ in reqs]
        cut1 = [300, 50, W]       # the third ends its first part exactly at the window's size
        cut2 = [560, 80, 200]
        rows = [[] for _ in reqs]

        def run(spans):
            steps = [SequenceStep(slots[i], reqs[i][a:b], list(range(b - a))) for i, a, b in spans]
            out = engine.step(steps).cpu().numpy()
            at = 0
            for i, a, b in spans:
                rows[i].append(out[at:at + b - a])
                at += b - a

        run([(i, 0, cut1[i]) for i in range(3)])
        run([(i, cut1[i], cut2[i]) for i in range(3)])
        at = list(cut2)
        while any(at[i] < len(reqs[i]) for i in range(3)):
            live = [i for i in range(3) if at[i] < len(reqs[i])]
            run([(i, at[i], at[i] + 1) for i in live])
            for i in live:
                at[i] += 1
        for i in range(3):
            engine.close_sequence(slots[i])
            tiny.assert_logits_close(np.concatenate(rows[i]), want[i], dtype,
                                     f"windowed, in parts, request {i}")
        engine.cache.table.check()
        assert engine.cache.table.slots.held == 0
        # a step that cannot fit is refused whole, before any portion ran
        s = engine.open_sequence()
        with pytest.raises(ValueError, match="positions"):
            engine.step([SequenceStep(s, [1] * 641, [])])
        assert engine.cache.length(s) == 0
        engine.close_sequence(s)
    finally:
        unregister_architecture("ToyWindowForCausalLM")


@pytest.mark.parametrize("name", ["tiny_a", "tiny_b"])
def test_single_token_steps_fold_the_norms_into_the_projections(tmp_path, monkeypatch, name):
    """In single-token steps the norm between two parts is work of the
    projections around it: only the first layer's first norm and the final norm
    still run as kernels. The logits agree with the plain model either way, and
    the two ways agree with each other."""
    import foundry_b200 as fb
    from foundry_b200.engine import SequenceStep
    from foundry_b200.kernels import ops
    folder = tiny.write_folder(str(tmp_path / name), name)
    cfg, w = plain.read_model(folder)
    reqs = [tiny.random_tokens(500 + i, n, cfg["vocab_size"]) for i, n in enumerate((33, 9, 20))]
    want = [plain.forward(cfg, w, r).numpy() for r in reqs]
    logits = {}
    for fused in (True, False):
        monkeypatch.setattr(ops, "NORM_FUSION", fused)
        engine = fb.Engine.from_folder(folder, dtype="bfloat16", max_tokens=512, max_slots=4)
        engine.use_graphs = False
        slots = [engine.open_sequence() for _ in reqs]
        engine.step([SequenceStep(s, r[:-4], []) for s, r in zip(slots, reqs)])
        rows = [[] for _ in reqs]
        for k in range(4, 0, -1):
            ops.PROFILER.start("steps")
            out = engine.step([SequenceStep(s, [r[-k]], [0]) for s, r in zip(slots, reqs)])
            counts = ops.PROFILER.take()["kernels"]
            ops.PROFILER.start(None)
            norms = sum(v["dispatch_count"] for key, v in counts.items() if key.startswith("add_rmsnorm"))
            layers = cfg["num_hidden_layers"]
            assert norms == (2 if fused else 2 * layers + 1), counts
            for i in range(len(reqs)):
                rows[i].append(out[i:i + 1].cpu().numpy())
        for i, r in enumerate(reqs):
            got = np.concatenate(rows[i])
            tiny.assert_logits_close(got, want[i][-4:], "bfloat16", f"{name} fused={fused} request {i}")
        logits[fused] = np.concatenate([np.concatenate(x) for x in rows])
    scale = float(np.abs(logits[False]).max())
    assert float(np.abs(logits[True] - logits[False]).max()) <= 0.03 * scale
