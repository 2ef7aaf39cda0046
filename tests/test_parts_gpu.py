"""Each part alone, and models put together from parts in ways Llama does not use: a run list that names a layer
twice, a layer that reads another layer's cache, a windowed attention group beside a full one, and a toy mixer with
a state of its own that is defined and registered here, without any change to the package (GPU)."""

import math

import numpy as np
import pytest
import torch

import helpers
import plain_model

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda")


def close(got, want, dtype):
    tol = 1e-4 if dtype == torch.float32 else 3e-2
    scale = float(want.abs().max())
    assert float((got.float().cpu() - want.float().cpu()).abs().max()) <= tol * max(scale, 1e-6), \
        (float((got.float().cpu() - want.float().cpu()).abs().max()), scale)


def fake_ctx(dtype, t=1):
    from prefixserve_b200.parts import StepContext
    z = torch.zeros(t, dtype=torch.int32, device=DEV)
    return StepContext(num_tokens=t, num_items=1, compute_dtype=dtype, device=DEV, items=[], token_ids=z, positions=z,
                       token_item=z, item_start=z, kv_len=z, slots=z, block_tables={}, max_new_tokens=t, max_kv_len=t,
                       all_decode=False)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_part(dtype):
    from prefixserve_b200.parts import make
    from prefixserve_b200.config import part
    norm = make("norm", part("rms", size=72, eps=1e-4))
    assert list(norm.param_specs()) == ["weight"] and norm.param_specs()["weight"].role == "vector"
    gain = 1 + 0.2 * torch.randn(72)
    norm.load({"weight": gain.to(DEV)}, compute_dtype=dtype, device=DEV)
    h = torch.randn(9, 72, device=DEV)
    delta = torch.randn(9, 72, device=DEV).to(dtype)
    want = plain_model.rms_norm((h + delta.float()).cpu(), gain, 1e-4)
    x = norm.forward(h, delta, fake_ctx(dtype, 9))
    assert x.dtype == dtype
    close(x, want, dtype)


def test_position_part_matches_plain_tables():
    from prefixserve_b200.parts import make
    from prefixserve_b200.config import part
    cfg = {"num_attention_heads": 2, "hidden_size": 64, "head_dim": 32, "rope_theta": 500000.0,
           "rope_scaling": {"rope_type": "llama3", "factor": 4.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                            "original_max_position_embeddings": 64}}
    pos = make("position", part("rope", head_dim=32, theta=500000.0, layout="half",
                                scaling={"kind": "llama3", "factor": 4.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                                         "original_max_positions": 64}))
    pos.prepare(max_positions=300, compute_dtype=torch.float32, device=DEV)
    cos, sin = plain_model.rope_tables(cfg, torch.arange(300), torch.float32)
    assert torch.equal(pos.cos[:300].cpu(), cos[:, :16]) and torch.equal(pos.sin[:300].cpu(), sin[:, :16])
    assert pos.cos.dtype == torch.float32
    none = make("position", part("none"))
    assert none.cos is None and not none.rotates
    assert make("position", part("rope", head_dim=32, theta=1.0, layout="interleaved", rotary_dim=16)).rotary_dim == 16
    with pytest.raises(ValueError):
        make("position", part("rope", head_dim=32, theta=1.0, layout="spiral"))
    with pytest.raises(ValueError):
        make("position", part("rope", head_dim=32, theta=1.0, rotary_dim=34))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_ffn_embedding_and_head_parts(dtype):
    from prefixserve_b200.parts import make
    from prefixserve_b200.config import part
    ffn = make("ffn", part("gated_mlp", hidden_size=40, intermediate_size=56, activation="silu"))
    w = {k: (0.3 * torch.randn(*s.shape)).to(dtype) for k, s in ffn.param_specs().items()}
    ffn.load({k: v.to(DEV) for k, v in w.items()}, compute_dtype=dtype, device=DEV)
    x = torch.randn(11, 40).to(dtype)
    want = plain_model.gated_mlp(x.float(), w["gate_proj"].float(), w["up_proj"].float(), w["down_proj"].float())
    close(ffn.forward(x.to(DEV), fake_ctx(dtype, 11)), want, dtype)
    with pytest.raises(ValueError):
        make("ffn", part("gated_mlp", hidden_size=4, intermediate_size=4, activation="gelu"))

    emb = make("embedding", part("token_embedding", vocab_size=33, hidden_size=40))
    table = torch.randn(33, 40).to(dtype)
    emb.load({"weight": table.to(DEV)}, compute_dtype=dtype, device=DEV)
    ids = torch.tensor([0, 32, 5, 5], dtype=torch.int32, device=DEV)
    assert torch.equal(emb.forward(ids).cpu(), table[[0, 32, 5, 5]].float())

    head = make("head", part("lm_head", vocab_size=33, hidden_size=40, tied=True))
    assert head.param_specs() == {}
    head.tie(emb.table)
    logits = head.forward(x[:3].to(DEV))
    assert logits.dtype == torch.float32
    close(logits, x[:3].float() @ table.float().t(), dtype)


# ---- whole models from parts -------------------------------------------------------------------------

def build(spec, dtype, seed=0, pages=64, std=0.15, stored=torch.float32):
    """``stored``: the type the "checkpoint" holds; matrices stored in float32 stay float32 in a bfloat16 run (and take
    the float32 product), stored in bfloat16 they run on the bfloat16 kernels.  ``raw`` comes back in float32."""
    from prefixserve_b200.cache import CacheManager
    from prefixserve_b200.engine import ModelRunner
    from prefixserve_b200.parts import build_model
    from prefixserve_b200.weights import convert_tensors, random_tensors
    model = build_model(spec)
    table = model.param_table()
    raw = random_tensors(table, seed, std=std, gain_noise=0.1, dtype=stored)
    model.load(convert_tensors(raw, table, compute_dtype=dtype, device=DEV), compute_dtype=dtype, device=DEV, max_positions=512)
    cache = CacheManager(model.cache_needs(), num_pages=pages, num_slots=4, max_seq_len=512, dtype=dtype, device=DEV,
                         enable_prefix_cache=False)
    return model, {k: v.float() for k, v in raw.items()}, cache, ModelRunner(model, cache, device=DEV)


def run_cut(runner, cache, tokens, cuts):
    """Feeds one request in portions; returns logits of every position."""
    from prefixserve_b200.engine import StepItem
    slot = cache.open()
    rows, at = [], 0
    for n in cuts:
        n = min(n, len(tokens) - at)
        if n <= 0:
            break
        assert cache.reserve(slot, at + n)
        rows.append(runner.step([StepItem(slot, at, np.asarray(tokens[at:at + n], dtype=np.int32), tuple(range(n)))]).cpu())
        cache.advance(slot, at + n)
        at += n
    cache.close(slot)
    cache.check()
    return torch.cat(rows)


def attn_spec(h, hq, hkv, d, window=None, own_kv=True, rope=True):
    from prefixserve_b200.config import part
    position = part("rope", head_dim=d, theta=10000.0, scaling=None, layout="half") if rope else part("none")
    return part("attention", hidden_size=h, num_heads=hq, num_kv_heads=hkv, head_dim=d, position=position, window=window,
                own_kv=own_kv)


def plain_attention_layer(x, w, prefix, hq, hkv, d, window, kv_from=None, rope=True):
    """Returns (output, (k, v)); with kv_from the layer has no key/value projection and reads the given ones."""
    t = x.shape[0]
    q = (x @ w[prefix + "q_proj"].t()).view(t, hq, d)
    cfg = {"num_attention_heads": hq, "hidden_size": hq * d, "head_dim": d, "rope_theta": 10000.0}
    cos, sin = plain_model.rope_tables(cfg, torch.arange(t), torch.float32)
    cos, sin = cos[:, None, :], sin[:, None, :]
    if rope:
        q = plain_model.apply_rope(q, cos, sin)
    if kv_from is None:
        k = (x @ w[prefix + "k_proj"].t()).view(t, hkv, d)
        if rope:
            k = plain_model.apply_rope(k, cos, sin)
        v = (x @ w[prefix + "v_proj"].t()).view(t, hkv, d)
    else:
        k, v = kv_from
    o = plain_model.causal_attention(q, k, v, window=window)
    return o.reshape(t, hq * d) @ w[prefix + "o_proj"].t(), (k, v)


def plain_forward(spec, w, tokens, mixers, ffns=None):
    """Whole-sequence float32 forward of a model given as a run list; ``mixers[layer]`` computes that layer's mixer,
    ``ffns[layer]`` (where given) its feed-forward instead of the gated MLP."""
    x_ids = torch.tensor(tokens)
    h = w["embedding.weight"][x_ids]
    kept = {}
    for call in spec.schedule:
        p = f"layers.{call.layer}."
        layer = spec.layers[call.layer]
        x = plain_model.rms_norm(h, w[p + "mixer_norm.weight"], layer.mixer_norm["eps"])
        out, keep = mixers[call.layer](x, w, p + "mixer.", kept.get(call.cache) if not call.writes_cache else None)
        if call.writes_cache:
            kept[call.cache] = keep
        h = h + out
        x = plain_model.rms_norm(h, w[p + "ffn_norm.weight"], layer.ffn_norm["eps"])
        if ffns and call.layer in ffns:
            h = h + ffns[call.layer](x, w, p + "ffn.")
        else:
            h = h + plain_model.gated_mlp(x, w[p + "ffn.gate_proj"], w[p + "ffn.up_proj"], w[p + "ffn.down_proj"])
    h = plain_model.rms_norm(h, w["final_norm.weight"], spec.final_norm["eps"])
    head = w["embedding.weight"] if spec.head["tied"] else w["head.weight"]
    return h @ head.t()


def toy_model_spec(layers, schedule, h=48, vocab=97):
    from prefixserve_b200.config import ModelSpec, part
    return ModelSpec(architecture="ToyFromParts", vocab_size=vocab, hidden_size=h, max_positions=512,
                     embedding=part("token_embedding", vocab_size=vocab, hidden_size=h), layers=tuple(layers),
                     schedule=tuple(schedule), final_norm=part("rms", size=h, eps=1e-5),
                     head=part("lm_head", vocab_size=vocab, hidden_size=h, tied=False))


def layer_of(mixer, h=48, inter=64, eps=1e-5):
    from prefixserve_b200.config import LayerSpec, part
    return LayerSpec(mixer=mixer, ffn=part("gated_mlp", hidden_size=h, intermediate_size=inter, activation="silu"),
                     mixer_norm=part("rms", size=h, eps=eps), ffn_norm=part("rms", size=h, eps=eps * 3))


CUTS = [[200], [150] + [1] * 50, [7, 2, 16, 3, 2, 5, 17, 2, 31, 4] * 3]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_run_list_with_shared_weights_shared_cache_and_a_window(dtype):
    """Layer 0 (full attention) runs twice with a cache entry each; layer 1 (window 24, no rotation) has a group of
    pages of its own; layer 2 has no key/value projection and reads the cache entry layer 0 wrote first."""
    from prefixserve_b200.config import LayerCall
    h, hq, hkv, d = 48, 3, 1, 16
    layers = [layer_of(attn_spec(h, hq, hkv, d)), layer_of(attn_spec(h, 2, 2, 32, window=24, rope=False)),
              layer_of(attn_spec(h, hq, hkv, d, own_kv=False))]
    schedule = [LayerCall(0, 0), LayerCall(1, 1), LayerCall(0, 2), LayerCall(2, 0, writes_cache=False)]
    spec = toy_model_spec(layers, schedule)
    model, raw, cache, runner = build(spec, dtype)
    assert len(cache.groups) == 2 and cache.entry_group == [0, 1, 0]
    assert "layers.2.mixer.k_proj" not in model.param_table()
    mixers = {
        0: lambda x, w, p, kv: plain_attention_layer(x, w, p, hq, hkv, d, None),
        1: lambda x, w, p, kv: plain_attention_layer(x, w, p, 2, 2, 32, 24, rope=False),
        2: lambda x, w, p, kv: plain_attention_layer(x, w, p, hq, hkv, d, None, kv_from=kv),
    }
    tokens = helpers.random_tokens(97, 200, seed=5)
    want = plain_forward(spec, raw, tokens, mixers)
    for cuts in CUTS:
        got = run_cut(runner, cache, tokens, cuts)
        if dtype == torch.float32:
            close(got, want, dtype)
        else:
            assert helpers.rel_err(got, want) < 0.05
    assert cache.free_pages(0) == 64 and cache.free_pages(1) == 64


@pytest.mark.parametrize("window", [50, 114, 16, 33])
def test_windowed_heads_of_64_decoded_through_captured_steps(window):
    """A window on the tensor-core decode kernel, token by token through a captured and replayed step: the keys an
    item reads run from the 16-aligned start of its window, so their number depends on (length - window) mod 16 and
    the captured launch must have room for the longest such span.  The sweep covers every residue (the kernel alone,
    with keys that make a short range show, is in the kernel tests)."""
    from prefixserve_b200.config import LayerCall
    from prefixserve_b200.ops import library
    h, hq, hkv, d = 128, 4, 2, 64
    spec = toy_model_spec([layer_of(attn_spec(h, hq, hkv, d, window=window), h=h, inter=96)], [LayerCall(0, 0)], h=h)
    model, raw, cache, runner = build(spec, torch.bfloat16, std=0.3, stored=torch.bfloat16)
    mixers = {0: lambda x, w, p, kv: plain_attention_layer(x, w, p, hq, hkv, d, window)}
    tokens = helpers.random_tokens(97, window + 70, seed=8)
    want = plain_forward(spec, raw, tokens, mixers)
    before = library.launch_counts["attention_decode"]
    got = run_cut(runner, cache, tokens, [1] * len(tokens))
    assert runner.graph_replays >= len(tokens) - 2 and library.launch_counts["attention_decode"] - before >= len(tokens) - 1
    assert helpers.rel_err(got, want) < 0.05
    # the same token by token without captured steps (launch shapes from each step's own lengths): the same to rounding
    model2, _, cache2, runner2 = build(spec, torch.bfloat16, std=0.3, stored=torch.bfloat16)
    runner2.use_graphs = False
    eager = run_cut(runner2, cache2, tokens, [1] * len(tokens))
    assert runner2.graph_replays == 0
    assert float((got - eager).abs().max()) <= 2e-2 * float(want.abs().max())


# ---- a toy mixer with a state of its own, defined here ---------------------------------------------------

DECAY = 0.6


def register_toy():
    from prefixserve_b200 import ops
    from prefixserve_b200.parts import CacheNeed, FixedState, Mixer, ParamSpec, register_mixer

    class DecayingSum(Mixer):
        """s_t = DECAY * s_(t-1) + x_t per request (float32 state [H] in the request's slot); y_t = s_t W^T."""

        def __init__(self, params):
            super().__init__(params)
            self.h = int(params["hidden_size"])

        def param_specs(self):
            return {"mix": ParamSpec((self.h, self.h))}

        def cache_need(self):
            return CacheNeed(state=FixedState((self.h,), torch.float32))

        def load(self, tensors, *, compute_dtype, device):
            self.w = tensors["mix"].contiguous()

        def forward(self, x, ctx, cache):
            s_all = torch.empty(x.shape, dtype=torch.float32, device=x.device)
            for item in ctx.items:  # a state is carried from where the request's last step left it
                s = cache.state[item.slot]
                n = item.end - item.start
                for j in range(n):
                    s = DECAY * s + x[item.first_token + j].float()
                    s_all[item.first_token + j] = s
                cache.state[item.slot] = s
            return ops.linear(s_all.to(x.dtype), self.w)

    register_mixer("decaying_sum", DecayingSum, replace=True)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_toy_mixer_with_state_is_registered_built_and_stepped(dtype):
    from prefixserve_b200.config import LayerCall, part
    from prefixserve_b200.engine import StepItem
    register_toy()
    h = 48
    layers = [layer_of(attn_spec(h, 3, 3, 16)), layer_of(part("decaying_sum", hidden_size=h))]
    spec = toy_model_spec(layers, [LayerCall(0, 0), LayerCall(1, 1)])
    model, raw, cache, runner = build(spec, dtype, seed=4, std=0.1)
    assert cache.entry_group == [0, None] and cache.state[1].shape == (4, h) and not cache.prefix_cache_possible

    def toy(x, w, p, kv):
        s = torch.zeros(h)
        out = []
        for t in range(x.shape[0]):
            s = DECAY * s + x[t]
            out.append(s)
        return torch.stack(out) @ w[p + "mix"].t(), None

    mixers = {0: lambda x, w, p, kv: plain_attention_layer(x, w, p, 3, 3, 16, None), 1: toy}
    seqs = [helpers.random_tokens(97, n, seed=20 + n) for n in (60, 45)]
    wants = [plain_forward(spec, raw, s, mixers) for s in seqs]
    for cuts in ([60], [40] + [1] * 20, [7, 2, 16, 3, 2, 5, 17, 2, 6]):
        for toks, want in zip(seqs, wants):
            got = run_cut(runner, cache, toks, cuts)  # the slot is reused: its state must start from zero again
            if dtype == torch.float32:
                close(got, want, dtype)
            else:
                assert helpers.rel_err(got, want) < 0.05
    # two requests interleaved in one batch keep their states apart
    a, b = cache.open(), cache.open()
    rows = {a: [], b: []}
    pa = pb = 0
    for na, nb in ((5, 1), (1, 9), (20, 1), (1, 1), (33, 33)):
        items = []
        for slot, toks, at, n in ((a, seqs[0], pa, na), (b, seqs[1], pb, nb)):
            n = min(n, len(toks) - at)
            cache.reserve(slot, at + n)
            items.append(StepItem(slot, at, np.asarray(toks[at:at + n], dtype=np.int32), tuple(range(n))))
        out = runner.step(items).cpu()
        rows[a].append(out[: len(items[0].tokens)])
        rows[b].append(out[len(items[0].tokens):])
        pa, pb = pa + len(items[0].tokens), pb + len(items[1].tokens)
        cache.advance(a, pa), cache.advance(b, pb)
    for slot, want in ((a, wants[0]), (b, wants[1])):
        got = torch.cat(rows[slot])
        if dtype == torch.float32:
            close(got, want[: got.shape[0]], dtype)
        else:
            assert helpers.rel_err(got, want[: got.shape[0]]) < 0.05


# ---- a toy feed-forward with routing and a toy position encoding, both defined here -------------------------

EXPERTS = 3


def register_toy_ffn_and_position():
    from prefixserve_b200 import ops
    from prefixserve_b200.parts import FeedForward, ParamSpec, PositionEncoding, register_ffn, register_position

    class RoutedMLP(FeedForward):
        """Each token goes to the one expert whose router score is highest (scores in float32); an expert is a small
        SiLU-gated MLP.  Routing lives inside the part: cache, scheduler and step function know nothing of it."""

        def __init__(self, params):
            super().__init__(params)
            self.h, self.inter, self.experts = int(params["hidden_size"]), int(params["intermediate_size"]), int(params["experts"])

        def param_specs(self):
            specs = {"router": ParamSpec((self.experts, self.h))}
            for e in range(self.experts):
                specs[f"experts.{e}.gate_up"] = ParamSpec((2 * self.inter, self.h))
                specs[f"experts.{e}.down"] = ParamSpec((self.h, self.inter))
            return specs

        def load(self, tensors, *, compute_dtype, device):
            self.router = tensors["router"].float().contiguous()
            self.gate_up = [tensors[f"experts.{e}.gate_up"].contiguous() for e in range(self.experts)]
            self.down = [tensors[f"experts.{e}.down"].contiguous() for e in range(self.experts)]

        def forward(self, x, ctx):
            choice = ops.linear(x.float().contiguous(), self.router).argmax(-1)   # float32 product on the CUDA cores
            out = torch.zeros_like(x)
            for e in range(self.experts):
                rows = (choice == e).nonzero().flatten()
                if rows.numel():
                    out[rows] = ops.linear(ops.gated_linear(x[rows].contiguous(), self.gate_up[e]), self.down[e])
            return out

    class LinearAngles(PositionEncoding):
        """Rotation by angles that grow linearly with the pair index instead of geometrically."""
        rotates = True

        def __init__(self, params):
            super().__init__(params)
            self.head_dim, self.step = int(params["head_dim"]), float(params["step"])
            self.cos = self.sin = None

        def prepare(self, *, max_positions, compute_dtype, device):
            angles = torch.outer(torch.arange(max_positions).float(), toy_frequencies(self.head_dim, self.step))
            self.cos, self.sin = angles.cos().to(device).contiguous(), angles.sin().to(device).contiguous()

    register_ffn("routed_mlp", RoutedMLP, replace=True)
    register_position("linear_angles", LinearAngles, replace=True)


def toy_frequencies(head_dim, step):
    return step * (1 + torch.arange(head_dim // 2).float())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_toy_routed_feed_forward_and_toy_positions(dtype):
    """A feed-forward with routing and a position encoding of another kind are registered from here, built by the
    framework's own builder, and stepped under every cutting: no file of the framework changes for them."""
    from prefixserve_b200.config import LayerCall, LayerSpec, part
    register_toy_ffn_and_position()
    h, hq, hkv, d, inter = 48, 3, 1, 16, 32
    mixer = part("attention", hidden_size=h, num_heads=hq, num_kv_heads=hkv, head_dim=d, window=None, own_kv=True,
                 position=part("linear_angles", head_dim=d, step=0.05))
    routed = LayerSpec(mixer=mixer, ffn=part("routed_mlp", hidden_size=h, intermediate_size=inter, experts=EXPERTS),
                       mixer_norm=part("rms", size=h, eps=1e-5), ffn_norm=part("rms", size=h, eps=1e-5))
    spec = toy_model_spec([routed, layer_of(attn_spec(h, hq, hkv, d))], [LayerCall(0, 0), LayerCall(1, 1)])
    model, raw, cache, runner = build(spec, dtype, seed=8, std=0.2)
    assert "layers.0.ffn.experts.2.down" in model.param_table() and "layers.0.ffn.router" in model.param_table()

    def toy_attention(x, w, p, kv):
        t = x.shape[0]
        angles = torch.outer(torch.arange(t).float(), toy_frequencies(d, 0.05))
        angles = torch.cat((angles, angles), dim=-1)  # the plain rotation takes tables of the full head size
        cos, sin = angles.cos()[:, None, :], angles.sin()[:, None, :]
        q = plain_model.apply_rope((x @ w[p + "q_proj"].t()).view(t, hq, d), cos, sin)
        k = plain_model.apply_rope((x @ w[p + "k_proj"].t()).view(t, hkv, d), cos, sin)
        v = (x @ w[p + "v_proj"].t()).view(t, hkv, d)
        return plain_model.causal_attention(q, k, v).reshape(t, hq * d) @ w[p + "o_proj"].t(), (k, v)

    def toy_ffn(x, w, p):
        choice = (x @ w[p + "router"].t()).argmax(-1)
        out = torch.zeros_like(x)
        for e in range(EXPERTS):
            gate, up = w[p + f"experts.{e}.gate_up"][:inter], w[p + f"experts.{e}.gate_up"][inter:]
            y = plain_model.gated_mlp(x, gate, up, w[p + f"experts.{e}.down"])
            out[choice == e] = y[choice == e]
        return out

    mixers = {0: toy_attention, 1: lambda x, w, p, kv: plain_attention_layer(x, w, p, hq, hkv, d, None)}
    tokens = helpers.random_tokens(97, 120, seed=31)
    want = plain_forward(spec, raw, tokens, mixers, ffns={0: toy_ffn})
    used = (plain_model.rms_norm(raw["embedding.weight"][torch.tensor(tokens)], raw["layers.0.mixer_norm.weight"], 1e-5)).shape
    assert used == (120, h)
    for cuts in ([120], [100] + [1] * 20, [7, 2, 16, 3, 2, 5, 17, 2, 31, 4, 40]):
        got = run_cut(runner, cache, tokens, cuts)
        if dtype == torch.float32:
            close(got, want, dtype)   # every token takes the same expert however the prompt is cut
        else:
            assert helpers.rel_err(got, want) < 0.08   # a near-tie at the router may pick another expert in bfloat16


# ---- other rotations, another activation, other block arrangements --------------------------------------

def register_partial_rotation():
    """A position part, defined here, that turns only the first ``rotary_dim`` elements of a head, in either pairing.
    It only describes its rotation (tables, rotary_dim, layout); the attention part and its kernels do the rest."""
    from prefixserve_b200.parts import PositionEncoding, register_position

    class PartialRotation(PositionEncoding):
        rotates = True

        def __init__(self, params):
            super().__init__(params)
            self.rotary_dim, self.layout, self.step = int(params["rotary_dim"]), params["layout"], float(params["step"])
            self.cos = self.sin = None

        def prepare(self, *, max_positions, compute_dtype, device):
            angles = torch.outer(torch.arange(max_positions).float(), toy_frequencies(self.rotary_dim, self.step))
            self.cos, self.sin = angles.cos().to(device).contiguous(), angles.sin().to(device).contiguous()

    register_position("partial_rotation", PartialRotation, replace=True)


def plain_partial_rotation(x, rotary_dim, layout, step):
    """x [T, heads, D] -> the first rotary_dim elements of every head turned by position, the rest untouched."""
    t = x.shape[0]
    angles = torch.outer(torch.arange(t).float(), toy_frequencies(rotary_dim, step))   # [T, rot/2]
    cos, sin = angles.cos()[:, None, :], angles.sin()[:, None, :]
    rot, rest = x[..., :rotary_dim], x[..., rotary_dim:]
    if layout == "half":
        x1, x2 = rot[..., : rotary_dim // 2], rot[..., rotary_dim // 2:]
        turned = torch.cat((x1 * cos - x2 * sin, x2 * cos + x1 * sin), dim=-1)
    else:
        x1, x2 = rot[..., 0::2], rot[..., 1::2]
        turned = torch.stack((x1 * cos - x2 * sin, x2 * cos + x1 * sin), dim=-1).flatten(-2)
    return torch.cat((turned, rest), dim=-1)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("d,rotary_dim,layout", [(64, 32, "half"), (64, 64, "interleaved"), (48, 20, "interleaved"), (128, 64, "half")])
def test_partial_and_interleaved_rotations_from_a_toy_part(dtype, d, rotary_dim, layout):
    """Head sizes at which the fused projections exist: a rotation they do not bake in must go round them (separate
    product, general rotary kernel, natural element order in the cache) and still agree with plain under every cutting."""
    from prefixserve_b200.config import LayerCall, part
    from prefixserve_b200.ops import library
    register_partial_rotation()
    h, hq, hkv = 96, 4, 2
    position = part("partial_rotation", rotary_dim=rotary_dim, layout=layout, step=0.03)
    mixer = part("attention", hidden_size=h, num_heads=hq, num_kv_heads=hkv, head_dim=d, window=None, own_kv=True, position=position)
    spec = toy_model_spec([layer_of(mixer, h=h, inter=64)], [LayerCall(0, 0)], h=h)
    model, raw, cache, runner = build(spec, dtype, seed=4, std=0.2, stored=dtype)
    assert model.blocks[0].mixer.paired is False and cache.needs[0].paged.key_order == "natural"

    def attention(x, w, p, kv):
        t = x.shape[0]
        q = plain_partial_rotation((x @ w[p + "q_proj"].t()).view(t, hq, d), rotary_dim, layout, 0.03)
        k = plain_partial_rotation((x @ w[p + "k_proj"].t()).view(t, hkv, d), rotary_dim, layout, 0.03)
        v = (x @ w[p + "v_proj"].t()).view(t, hkv, d)
        return plain_model.causal_attention(q, k, v).reshape(t, hq * d) @ w[p + "o_proj"].t(), (k, v)

    tokens = helpers.random_tokens(97, 150, seed=12)
    want = plain_forward(spec, raw, tokens, {0: attention})
    before = library.launch_counts.copy()
    for cuts in ([150], [110] + [1] * 40, [7, 2, 16, 3, 2, 5, 17, 2, 31, 4, 61]):
        got = run_cut(runner, cache, tokens, cuts)
        if dtype == torch.float32:
            close(got, want, dtype)
        else:
            assert helpers.rel_err(got, want) < 0.05
    taken = library.launch_counts - before
    assert taken["rope_append"] > 0 and taken["gemm_stream_norm_rope"] == 0 and taken["gemm_tcgen05_rope"] == 0, dict(taken)


def test_a_reader_with_another_element_order_is_refused():
    """A layer that reads another layer's keys must keep a head's elements in the order the writer used."""
    from prefixserve_b200.config import LayerCall, part
    from prefixserve_b200.parts import build_model
    register_partial_rotation()
    h, hq, hkv, d = 96, 4, 2, 64
    partial = part("attention", hidden_size=h, num_heads=hq, num_kv_heads=hkv, head_dim=d, window=None, own_kv=True,
                   position=part("partial_rotation", rotary_dim=32, layout="half", step=0.03))
    reader = attn_spec(h, hq, hkv, d, own_kv=False)   # whole-head rotation: pair-interleaved order
    spec = toy_model_spec([layer_of(partial, h=h), layer_of(reader, h=h)], [LayerCall(0, 0), LayerCall(1, 0, writes_cache=False)], h=h)
    with pytest.raises(ValueError, match="reads cache entry"):
        build_model(spec).cache_needs()


def gelu_mlp(x, gate_w, up_w, down_w):
    gate = x @ gate_w.t()
    return (torch.nn.functional.gelu(gate, approximate="tanh") * (x @ up_w.t())) @ down_w.t()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("arrangement", ["pre_norm", "parallel"])
def test_another_activation_and_the_parallel_arrangement(dtype, arrangement):
    """gated_mlp with the tanh form of GELU (in every kernel that applies the activation: cuts of 1, of a few and of
    hundreds of tokens), a block whose sublayers both read the entering stream, and a layer that only mixes."""
    from prefixserve_b200.config import LayerCall, LayerSpec, part
    from prefixserve_b200.ops import library, tensorcore
    h, hq, hkv, d, inter = 128, 2, 1, 64, 256
    norm = part("rms", size=h, eps=1e-5)
    gelu = LayerSpec(mixer=attn_spec(h, hq, hkv, d), ffn=part("gated_mlp", hidden_size=h, intermediate_size=inter, activation="gelu_tanh"),
                     mixer_norm=norm, ffn_norm=norm, arrangement=arrangement)
    only_mixer = LayerSpec(mixer=attn_spec(h, hq, hkv, d), ffn=None, mixer_norm=norm, ffn_norm=None, arrangement=arrangement)
    spec = toy_model_spec([gelu, only_mixer, gelu], [LayerCall(0, 0), LayerCall(1, 1), LayerCall(2, 2)], h=h)
    model, raw, cache, runner = build(spec, dtype, seed=6, std=0.1, stored=dtype)
    assert "layers.1.ffn.gate_proj" not in model.param_table() and "layers.2.ffn.gate_proj" in model.param_table()

    def forward(tokens):
        w = raw
        hh = w["embedding.weight"][torch.tensor(tokens)]
        for i in range(3):
            p = f"layers.{i}."
            x = plain_model.rms_norm(hh, w[p + "mixer_norm.weight"], 1e-5)
            mixed, _ = plain_attention_layer(x, w, p + "mixer.", hq, hkv, d, None)
            if i == 1:
                hh = hh + mixed
                continue
            if arrangement == "pre_norm":
                hh = hh + mixed
                x2 = plain_model.rms_norm(hh, w[p + "ffn_norm.weight"], 1e-5)
                hh = hh + gelu_mlp(x2, w[p + "ffn.gate_proj"], w[p + "ffn.up_proj"], w[p + "ffn.down_proj"])
            else:
                x2 = plain_model.rms_norm(hh, w[p + "ffn_norm.weight"], 1e-5)
                hh = hh + mixed + gelu_mlp(x2, w[p + "ffn.gate_proj"], w[p + "ffn.up_proj"], w[p + "ffn.down_proj"])
        return plain_model.rms_norm(hh, w["final_norm.weight"], 1e-5) @ w["head.weight"].t()

    tokens = helpers.random_tokens(97, 400, seed=3)
    want = forward(tokens)
    tiles, rows = tensorcore.TCGEN05_MIN_TILES, tensorcore.TCGEN05_MIN_ROWS
    tensorcore.TCGEN05_MIN_TILES = tensorcore.TCGEN05_MIN_ROWS = 1     # let the portions take the tcgen05 product with the fused activation
    before = library.launch_counts.copy()
    try:
        for cuts in ([400], [300, 40] + [1] * 60, [7, 2, 16, 3, 2, 5, 17, 2, 31, 4] * 5):
            got = run_cut(runner, cache, tokens, cuts)
            if dtype == torch.float32:
                close(got, want, dtype)
            else:
                assert helpers.rel_err(got, want) < 0.05
    finally:
        tensorcore.TCGEN05_MIN_TILES, tensorcore.TCGEN05_MIN_ROWS = tiles, rows
    taken = library.launch_counts - before
    if dtype == torch.bfloat16:
        fused = "gemm_stream_norm_gated" if arrangement == "pre_norm" else "gemm_stream_gated"
        assert taken["gemm_tcgen05_gated"] > 0 and taken[fused] > 0, dict(taken)
    if arrangement == "parallel":
        assert taken["residual_add"] > 0


def test_unknown_activation_and_arrangement_are_refused_before_anything_runs():
    from prefixserve_b200 import ops
    from prefixserve_b200.config import LayerSpec, part
    from prefixserve_b200.parts import Block
    with pytest.raises(ValueError, match="activation"):
        layer_of(attn_spec(48, 3, 1, 16)).ffn.with_params(activation="relu6") and Block(
            LayerSpec(mixer=attn_spec(48, 3, 1, 16), ffn=part("gated_mlp", hidden_size=48, intermediate_size=64, activation="relu6"),
                      mixer_norm=part("rms", size=48, eps=1e-5), ffn_norm=part("rms", size=48, eps=1e-5)))
    with pytest.raises(ValueError, match="arrangement"):
        Block(LayerSpec(mixer=attn_spec(48, 3, 1, 16), ffn=None, mixer_norm=part("rms", size=48, eps=1e-5), ffn_norm=None,
                        arrangement="sandwich"))
    x = torch.zeros(2, 64, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(ops.KernelError, match="activation"):
        ops.gated_linear(x, torch.zeros(32, 64, dtype=torch.bfloat16, device=DEV), "relu6")
    from prefixserve_b200.ops.library import lib
    assert lib().psb_gemm_stream_gated(x.data_ptr(), x.data_ptr(), x.data_ptr(), 2, 16, 64, 148, 7, None) != 0   # the C entry refuses too
