"""Each part alone against the plain implementation, a schedule that names a layer twice and lets a
call read another call's cache, and a toy mixer with state of its own that is registered, built and
stepped without a change to the framework's files."""
import dataclasses
import json

import pytest
import torch

import plain_llama
from conftest import TINY_B, TINY_C
from gpu_common import BF16_REL, F32_ATOL, F32_RTOL, need_gpu

pytestmark = pytest.mark.gpu
CUDA = torch.device("cuda")


def _batch(entries):
    """entries: (request id, slot, kv_start, q_len) -> StepBatch without tokens."""
    from torchinferno_b200.engine.batch import EntryPlacement, build_batch
    places, row = [], 0
    for rid, slot, start, n in entries:
        places.append(EntryPlacement(rid, slot, row, n, start))
        row += n
    batch, _ = build_batch(places, [[0] * p.q_len for p in places], [[] for _ in places], [], CUDA)
    return batch


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_part(dtype):
    need_gpu()
    from torchinferno_b200.parts.base import PartSpec, ResidualStream, build_part
    norm = build_part("norm", PartSpec("rmsnorm", {"width": 120, "eps": 3e-6}), dtype=dtype, device=CUDA)
    assert [(w.name, w.shape, w.init, w.role) for w in norm.weight_specs()] == [("weight", (120,), "ones", "vector")]
    w = 1 + 0.3 * torch.randn(120)
    norm.bind({"weight": w.to(torch.bfloat16).cuda()})
    w = w.to(torch.bfloat16).double()
    res = torch.randn(9, 120) * 2
    stream = ResidualStream(res.clone().cuda(), dtype)
    tol = dict(atol=2e-6, rtol=2e-6) if dtype == torch.float32 else dict(atol=2e-2, rtol=1e-2)
    assert torch.allclose(stream.normed(norm).cpu().double(), plain_llama.rms_norm(res.double(), w, 3e-6), **tol)
    delta = torch.randn(9, 120).to(dtype)
    stream.add(delta.cuda())
    with pytest.raises(RuntimeError):
        stream.add(delta.cuda())
    got = stream.normed(norm)
    assert stream.pending is None and torch.equal(stream.residual.cpu(), res + delta.float())
    assert torch.allclose(got.cpu().double(), plain_llama.rms_norm((res + delta.float()).double(), w, 3e-6), **tol)


def test_rotary_part_tables_match_the_plain_law():
    need_gpu()
    from torchinferno_b200.parts.base import PartSpec, build_part
    for cfg in (TINY_B, TINY_C, {**TINY_B, "rope_scaling": None}):
        d = cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"]
        rope = build_part("position", PartSpec("rotary", {"head_dim": d, "theta": cfg["rope_theta"], "scaling": cfg["rope_scaling"]}),
                          dtype=torch.float32, device=CUDA)
        assert torch.equal(rope.inv_freq.cpu(), plain_llama.inverse_frequencies(cfg))
    with pytest.raises(ValueError):
        build_part("position", PartSpec("rotary", {"head_dim": 32, "theta": 1e4, "scaling": {"rope_type": "yarn"}}), dtype=torch.float32, device=CUDA)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu_part(dtype):
    need_gpu()
    from torchinferno_b200.parts.base import LayerContext, PartSpec, build_part
    ffn = build_part("feed_forward", PartSpec("swiglu", {"hidden_size": 72, "intermediate_size": 200}), dtype=dtype, device=CUDA)
    assert {w.name: w.shape for w in ffn.weight_specs()} == {"gate_proj.weight": (200, 72), "up_proj.weight": (200, 72), "down_proj.weight": (72, 200)}
    ws = {"gate_proj.weight": torch.randn(200, 72) * 0.2, "up_proj.weight": torch.randn(200, 72) * 0.2, "down_proj.weight": torch.randn(72, 200) * 0.2}
    ws = {k: v.to(torch.bfloat16) for k, v in ws.items()}
    ffn.bind({k: v.to(dtype).cuda() for k, v in ws.items()})
    x = torch.randn(11, 72).to(dtype)
    got = ffn.forward(x.cuda(), LayerContext(batch=None))
    gate_w, up_w, down_w = (ws[k].double() for k in ("gate_proj.weight", "up_proj.weight", "down_proj.weight"))
    if dtype == torch.float32:
        want, tol = plain_llama.swiglu_mlp(x.double(), gate_w, up_w, down_w), dict(atol=1e-5, rtol=1e-5)
    else:
        # The part stores gate / up and their product in bfloat16 between its kernels.  With these weights an output is
        # a sum of 200 terms of size 1, so those roundings move it by up to 0.1 in absolute terms, whatever its own
        # size: the plain formula is therefore rounded at the same two places, and what is left to compare is the
        # arithmetic (fp32 sums in another order, the fast exponential) and the rounding of the result itself.
        as_stored = lambda t: t.to(torch.bfloat16).double()
        gate, up = as_stored(x.double() @ gate_w.T), as_stored(x.double() @ up_w.T)
        want = as_stored((gate / (1 + torch.exp(-gate))) * up) @ down_w.T
        tol = dict(atol=2e-2, rtol=8e-3)
    assert torch.allclose(got.cpu().double(), want, **tol), (got.cpu().double() - want).abs().max()


def _attention_weights(hidden, heads, kv, d, seed=0):
    g = torch.Generator().manual_seed(seed)
    mk = lambda *s: (torch.randn(*s, generator=g) * 0.3).to(torch.bfloat16)
    return {"q_proj.weight": mk(heads * d, hidden), "k_proj.weight": mk(kv * d, hidden), "v_proj.weight": mk(kv * d, hidden),
            "o_proj.weight": mk(hidden, heads * d)}


def _plain_attention(x, ws, heads, kv, d, cfg, window=None):
    T = x.shape[0]
    inv = plain_llama.inverse_frequencies(cfg)
    pos = torch.arange(T)
    q = plain_llama.rotary((x @ ws["q_proj.weight"].double().T).view(T, heads, d).transpose(0, 1), pos, inv)
    k = plain_llama.rotary((x @ ws["k_proj.weight"].double().T).view(T, kv, d).transpose(0, 1), pos, inv)
    v = (x @ ws["v_proj.weight"].double().T).view(T, kv, d).transpose(0, 1)
    a = plain_llama.causal_attention(q, k, v, heads // kv, window=window).transpose(0, 1).reshape(T, heads * d)
    return a @ ws["o_proj.weight"].double().T


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [None, 9])
def test_attention_part_in_portions_over_its_own_cache(dtype, window):
    need_gpu()
    from torchinferno_b200.cache.manager import CacheManager
    from torchinferno_b200.kernels import ops
    from torchinferno_b200.parts.base import KVBinding, LayerContext, PartSpec, build_part
    hidden, heads, kv, d = 120, 5, 1, 48
    cfg = {**TINY_C}
    position = PartSpec("rotary", {"head_dim": d, "theta": cfg["rope_theta"], "scaling": cfg["rope_scaling"]})
    mixer = build_part("mixer", PartSpec("gqa_attention", {"hidden_size": hidden, "heads": heads, "kv_heads": kv, "head_dim": d,
                                                            "position": position, "window": window}), dtype=dtype, device=CUDA)
    assert mixer.cache_spec().window == window and mixer.state_spec() is None
    ws = _attention_weights(hidden, heads, kv, d)
    mixer.bind({k: v.to(dtype).cuda() for k, v in ws.items()})
    cache = CacheManager([mixer.cache_spec()], [None], page_size=4, num_pages=40, max_requests=3, max_request_tokens=80,
                         dtype=dtype, device=CUDA)
    cache.groups[0].pool.fill_(float("nan"))
    x = (torch.randn(70, hidden) * 0.5).to(dtype)
    want = _plain_attention(x.double(), ws, heads, kv, d, cfg, window)
    cache.open("warm"), cache.extend("warm", 3)        # another request holds the first pages and slot
    outs, pos = [], 0
    for n in (1, 2, 30, 5, 1, 31):
        cache.open("r") if pos == 0 else None
        start = cache.extend("r", n)
        for group, (idx, val) in zip(cache.groups, cache.drain_table_updates()):
            if idx:
                ops.scatter_i32(group.table_device, torch.tensor(idx, dtype=torch.int32).cuda(), torch.tensor(val, dtype=torch.int32).cuda())
        b = cache.kv_binding(0)
        ctx = LayerContext(batch=_batch([("r", cache.slot("r"), start, n)]), kv=KVBinding(b.pool, b.block_table, b.page_size, b.window),
                           error_word=cache.error_word)
        outs.append(mixer.forward(x[pos:pos + n].cuda().contiguous(), ctx))
        cache.release_behind_window("r")
        pos += n
    assert int(cache.error_word) == 0
    if window:
        assert -1 in cache.block_table("r")               # pages behind the window went back
    got = torch.cat(outs).cpu().double()
    if dtype == torch.float32:
        assert torch.allclose(got, want, atol=2e-5, rtol=1e-4)
    else:
        assert (got - want).abs().max() <= BF16_REL * want.abs().max()


def test_a_layer_run_twice_and_a_call_that_reads_another_calls_cache(model_folders):
    need_gpu()
    from torchinferno_b200.config.model_config import LlamaConfig
    from torchinferno_b200.engine.batch import StepEntry
    from torchinferno_b200.engine.factory import make_runner
    from torchinferno_b200.models.llama import build_llama
    from torchinferno_b200.models.model import CausalLM
    from torchinferno_b200.models.spec import LayerCall
    from torchinferno_b200.weights.loader import load_weights
    folder = model_folders["B"]
    config, weights = plain_llama.read_model_folder(folder)
    spec = build_llama(LlamaConfig.from_dict(config))
    # layer 0, layer 1, layer 0 again (cache of its own), then layer 2 reading what layer 1 stored
    schedule = (LayerCall(0, 0), LayerCall(1, 1), LayerCall(0, 2), LayerCall(2, 1, writes_cache=False))
    model = CausalLM(dataclasses.replace(spec, schedule=schedule), dtype=torch.float32, device=CUDA)
    load_weights(model, folder)
    runner = make_runner(model, page_size=16, max_tokens=256, max_requests=2)
    tokens = torch.randint(0, config["vocab_size"], (90,), generator=torch.Generator().manual_seed(5)).tolist()

    # plain: the same order, with the shared cache spelled out
    def layer(x, i, kv_from=None):
        heads, kv = config["num_attention_heads"], config["num_key_value_heads"]
        d, eps, T = config["hidden_size"] // heads, config["rms_norm_eps"], x.shape[0]
        p, inv, pos = f"model.layers.{i}.", plain_llama.inverse_frequencies(config), torch.arange(T)
        n = plain_llama.rms_norm(x, weights[p + "input_layernorm.weight"], eps)
        q = plain_llama.rotary((n @ weights[p + "self_attn.q_proj.weight"].T).view(T, heads, d).transpose(0, 1), pos, inv)
        if kv_from is None:
            k = plain_llama.rotary((n @ weights[p + "self_attn.k_proj.weight"].T).view(T, kv, d).transpose(0, 1), pos, inv)
            v = (n @ weights[p + "self_attn.v_proj.weight"].T).view(T, kv, d).transpose(0, 1)
        else:
            k, v = kv_from
        a = plain_llama.causal_attention(q, k, v, heads // kv).transpose(0, 1).reshape(T, heads * d)
        x = x + a @ weights[p + "self_attn.o_proj.weight"].T
        n = plain_llama.rms_norm(x, weights[p + "post_attention_layernorm.weight"], eps)
        x = x + plain_llama.swiglu_mlp(n, weights[p + "mlp.gate_proj.weight"], weights[p + "mlp.up_proj.weight"], weights[p + "mlp.down_proj.weight"])
        return x, (k, v)

    x = weights["model.embed_tokens.weight"][torch.tensor(tokens)]
    x, _ = layer(x, 0)
    x, kv1 = layer(x, 1)
    x, _ = layer(x, 0)
    x, _ = layer(x, 2, kv_from=kv1)
    want = plain_llama.rms_norm(x, weights["model.norm.weight"], config["rms_norm_eps"]) @ weights["model.embed_tokens.weight"].T
    with torch.inference_mode():
        got = torch.cat([runner.step([StepEntry("a", tokens[:50], list(range(50)))]),
                         runner.step([StepEntry("a", tokens[50:52], [0, 1])]),
                         runner.step([StepEntry("a", tokens[52:], list(range(38)))])]).cpu().double()
    assert torch.allclose(got, want, atol=F32_ATOL, rtol=F32_RTOL), (got - want).abs().max()


# ------------------------------------------------------------------ toy mixer with state
def test_a_toy_mixer_with_state_of_its_own_is_registered_built_and_stepped(tmp_path):
    """A mixer defined here: y_t = W . mean(x_0 .. x_t).  It keeps no keys; its state (the running sum
    and the count) is of fixed size per request and lives in the cache manager's state slots.  It is
    registered as a part, named by a new architecture's model description beside an attention layer,
    given random weights by the framework's own writer, loaded, and stepped in portions."""
    need_gpu()
    from torchinferno_b200.config.registry import ArchitectureEntry, register_architecture, unregister_architecture
    from torchinferno_b200.engine.batch import StepEntry
    from torchinferno_b200.engine.factory import load_model, make_runner
    from torchinferno_b200.models.spec import BlockSpec, LayerCall, ModelSpec
    from torchinferno_b200.parts.base import Mixer, PartSpec, StateSpec, WeightSpec, register_part, unregister_part
    from torchinferno_b200.weights.random_init import write_random_model

    class RunningMeanMixer(Mixer):
        def __init__(self, *, width, dtype, device):
            super().__init__(dtype=dtype, device=device)
            self.width = width

        def weight_specs(self):
            return [WeightSpec("mix.weight", (self.width, self.width), std=0.2)]

        def bind(self, weights):
            self.weight = weights["mix.weight"].float()

        def state_spec(self):
            return StateSpec((self.width + 1,), torch.float32)      # running sum and count

        def forward(self, x, ctx):
            out = torch.empty_like(x)
            for e in ctx.batch.entries:                              # a request's tokens in order
                rows = slice(e.q_start, e.q_start + e.q_len)
                state = ctx.state[e.slot]
                sums = state[:-1] + torch.cumsum(x[rows].float(), dim=0)
                counts = state[-1] + torch.arange(1, e.q_len + 1, device=x.device)
                out[rows] = ((sums / counts[:, None]) @ self.weight.T).to(x.dtype)
                state[:-1], state[-1] = sums[-1], counts[-1]
            return out

    @dataclasses.dataclass(frozen=True)
    class ToyConfig:
        vocab_size: int
        width: int
        inter: int

        @classmethod
        def from_dict(cls, data):
            return cls(data["vocab_size"], data["width"], data["inter"])

    def build_toy(cfg):
        norm = PartSpec("rmsnorm", {"width": cfg.width, "eps": 1e-5})
        ffn = PartSpec("swiglu", {"hidden_size": cfg.width, "intermediate_size": cfg.inter}, prefix="ffn.")
        toy = PartSpec("prenorm", {"mixer": PartSpec("running_mean", {"width": cfg.width}, prefix="toy."), "feed_forward": ffn,
                                   "mixer_norm": dataclasses.replace(norm, prefix="n1."), "feed_forward_norm": dataclasses.replace(norm, prefix="n2.")})
        attn = PartSpec("prenorm", {"mixer": PartSpec("gqa_attention", {
            "hidden_size": cfg.width, "heads": 2, "kv_heads": 1, "head_dim": 16, "position": PartSpec("none", {"head_dim": 16})}, prefix="attn."),
            "feed_forward": ffn, "mixer_norm": dataclasses.replace(norm, prefix="n1."), "feed_forward_norm": dataclasses.replace(norm, prefix="n2.")})
        return ModelSpec(architecture="ToyForCausalLM", hidden_size=cfg.width, vocab_size=cfg.vocab_size, max_positions=512,
                         embedding_name="emb.weight", layers=(BlockSpec(toy, "l0."), BlockSpec(attn, "l1.")),
                         schedule=(LayerCall(0, None), LayerCall(1, 0), LayerCall(0, None)),
                         final_norm=dataclasses.replace(norm, prefix="final."), head_name="head.weight")

    register_part("mixer", "running_mean", RunningMeanMixer)
    register_architecture(ArchitectureEntry("ToyForCausalLM", ToyConfig, build_toy, model_types=("toy",)))
    try:
        cfg = {"architectures": ["ToyForCausalLM"], "model_type": "toy", "vocab_size": 50, "width": 24, "inter": 40}
        write_random_model(cfg, tmp_path, seed=11)
        model = load_model(tmp_path, dtype="float32")
        assert [s is not None for s in model.state_requirements()] == [True, False, True] and len(model.cache_requirements()) == 1
        runner = make_runner(model, page_size=4, max_tokens=128, max_requests=3)
        reqs = {"a": torch.randint(0, 50, (37,)).tolist(), "b": torch.randint(0, 50, (9,)).tolist()}
        with torch.inference_mode():
            whole = {k: runner.step([StepEntry(k + "w", v, list(range(len(v))))]).cpu() for k, v in reqs.items()}
            runner.end(["aw", "bw"])
            parts = {"a": [], "b": []}
            parts["a"].append(runner.step([StepEntry("a", reqs["a"][:5], list(range(5)))]).cpu())
            mixed = runner.step([StepEntry("b", reqs["b"][:8], list(range(8))), StepEntry("a", reqs["a"][5:6], [0])]).cpu()
            parts["b"].append(mixed[:8]), parts["a"].append(mixed[8:])
            mixed = runner.step([StepEntry("a", reqs["a"][6:], list(range(31))), StepEntry("b", reqs["b"][8:], [0])]).cpu()
            parts["a"].append(mixed[:31]), parts["b"].append(mixed[31:])
            runner.end(["a", "b"])
        for k in reqs:
            assert torch.allclose(torch.cat(parts[k]), whole[k], atol=1e-5, rtol=1e-4)
        # and the whole against plain arithmetic of the same description
        _, w = plain_llama.read_model_folder(tmp_path)
        def ffn(x, p):
            return plain_llama.swiglu_mlp(x, w[p + "ffn.gate_proj.weight"], w[p + "ffn.up_proj.weight"], w[p + "ffn.down_proj.weight"])
        def toy_layer(x):
            n = plain_llama.rms_norm(x, w["l0.n1.weight"], 1e-5)
            x = x + (torch.cumsum(n, 0) / torch.arange(1, len(n) + 1)[:, None]) @ w["l0.toy.mix.weight"].T
            return x + ffn(plain_llama.rms_norm(x, w["l0.n2.weight"], 1e-5), "l0.")
        def attn_layer(x):
            n, T = plain_llama.rms_norm(x, w["l1.n1.weight"], 1e-5), x.shape[0]
            q = (n @ w["l1.attn.q_proj.weight"].T).view(T, 2, 16).transpose(0, 1)
            k = (n @ w["l1.attn.k_proj.weight"].T).view(T, 1, 16).transpose(0, 1)
            v = (n @ w["l1.attn.v_proj.weight"].T).view(T, 1, 16).transpose(0, 1)
            x = x + plain_llama.causal_attention(q, k, v, 2).transpose(0, 1).reshape(T, 32) @ w["l1.attn.o_proj.weight"].T
            return x + ffn(plain_llama.rms_norm(x, w["l1.n2.weight"], 1e-5), "l1.")
        x = toy_layer(attn_layer(toy_layer(w["emb.weight"][torch.tensor(reqs["a"])])))
        want = plain_llama.rms_norm(x, w["final.weight"], 1e-5) @ w["head.weight"].T
        assert torch.allclose(whole["a"].double(), want, atol=2e-5, rtol=1e-4), (whole["a"].double() - want).abs().max()
    finally:
        unregister_part("mixer", "running_mean")
        unregister_architecture("ToyForCausalLM")


def test_a_toy_routed_feed_forward_and_a_toy_position_encoding_are_registered_and_stepped(tmp_path):
    """Two more parts defined here, neither known to the framework: a feed-forward that routes every token to
    the best of three small experts (router logits and the softmax weight in 32-bit), and a position encoding
    that scales queries by g(t) = 1.02^t and keys by 1 / g(s), so that a score is q.k g(t) / g(s).  One layer
    has the routed feed-forward and the toy encoding, the other the dense feed-forward and no encoding: parts
    are chosen layer by layer.  Stepped whole, in portions and mixed, against plain arithmetic."""
    need_gpu()
    from torchinferno_b200.config.registry import ArchitectureEntry, register_architecture, unregister_architecture
    from torchinferno_b200.engine.batch import StepEntry
    from torchinferno_b200.engine.factory import load_model, make_runner
    from torchinferno_b200.kernels import ops
    from torchinferno_b200.models.spec import BlockSpec, LayerCall, ModelSpec
    from torchinferno_b200.parts.base import (FeedForward, PartSpec, PositionEncoding, WeightSpec, register_part,
                                              unregister_part)
    from torchinferno_b200.weights.random_init import write_random_model
    EXPERTS, WIDTH, INTER, HEADS, KV, D, BASE = 3, 24, 16, 2, 1, 16, 1.02

    class RoutedFeedForward(FeedForward):
        def __init__(self, *, width, inter, experts, dtype, device):
            super().__init__(dtype=dtype, device=device)
            self.width, self.inter, self.experts = width, inter, experts

        def weight_specs(self):
            specs = [WeightSpec("router.weight", (self.experts, self.width), std=0.5)]
            for e in range(self.experts):
                specs += [WeightSpec(f"experts.{e}.up.weight", (self.inter, self.width), std=0.2),
                          WeightSpec(f"experts.{e}.down.weight", (self.width, self.inter), std=0.2)]
            return specs

        def bind(self, weights):
            self.router = weights["router.weight"].float()
            self.up = [weights[f"experts.{e}.up.weight"].float() for e in range(self.experts)]
            self.down = [weights[f"experts.{e}.down.weight"].float() for e in range(self.experts)]

        def forward(self, x, ctx):
            xf = x.float()
            prob = torch.softmax(xf @ self.router.T, dim=-1)
            weight, choice = prob.max(dim=-1)
            out = torch.zeros_like(xf)
            for e in range(self.experts):
                rows = (choice == e).nonzero().flatten()
                if rows.numel():
                    out[rows] = (torch.relu(xf[rows] @ self.up[e].T) @ self.down[e].T) * weight[rows, None]
            return out.to(x.dtype)

    class GeometricScaling(PositionEncoding):
        def __init__(self, *, head_dim, base, dtype, device):
            super().__init__(dtype=dtype, device=device)
            self.base = base
            self.none = torch.zeros(0, dtype=torch.float32, device=device)

        def encode_and_store(self, qkv, q_out, ctx, heads, kv_heads, head_dim):
            g = torch.pow(torch.tensor(self.base, device=qkv.device), ctx.batch.positions.float())[:, None]
            scaled = qkv.float().clone()
            scaled[:, :heads * head_dim] *= g
            scaled[:, heads * head_dim:(heads + kv_heads) * head_dim] /= g
            kv = ctx.kv
            # the framework's own kernel stores k and v in their pages (no rotation: rot_dim 0)
            return ops.rope_append(scaled.to(qkv.dtype), q_out, kv.pool, ctx.batch.positions, ctx.batch.token_slot, kv.block_table,
                                   self.none, heads, kv_heads, head_dim, rot_dim=0, write_kv=True, error_word=ctx.error_word)

    @dataclasses.dataclass(frozen=True)
    class ToyConfig:
        vocab_size: int

        @classmethod
        def from_dict(cls, data):
            return cls(data["vocab_size"])

    def build_toy(cfg):
        norm = PartSpec("rmsnorm", {"width": WIDTH, "eps": 1e-5})
        def attention(position):
            return PartSpec("gqa_attention", {"hidden_size": WIDTH, "heads": HEADS, "kv_heads": KV, "head_dim": D,
                                              "position": position}, prefix="attn.")
        norms = {"mixer_norm": dataclasses.replace(norm, prefix="n1."), "feed_forward_norm": dataclasses.replace(norm, prefix="n2.")}
        routed = PartSpec("prenorm", {"mixer": attention(PartSpec("geometric", {"head_dim": D, "base": BASE})),
                                      "feed_forward": PartSpec("toy_routed", {"width": WIDTH, "inter": INTER, "experts": EXPERTS}, prefix="moe."),
                                      **norms})
        dense = PartSpec("prenorm", {"mixer": attention(PartSpec("none", {"head_dim": D})),
                                     "feed_forward": PartSpec("swiglu", {"hidden_size": WIDTH, "intermediate_size": INTER}, prefix="ffn."),
                                     **norms})
        return ModelSpec(architecture="Toy2ForCausalLM", hidden_size=WIDTH, vocab_size=cfg.vocab_size, max_positions=256,
                         embedding_name="emb.weight", layers=(BlockSpec(routed, "l0."), BlockSpec(dense, "l1.")),
                         schedule=(LayerCall(0, 0), LayerCall(1, 1)),
                         final_norm=dataclasses.replace(norm, prefix="final."), head_name="head.weight")

    register_part("feed_forward", "toy_routed", RoutedFeedForward)
    register_part("position", "geometric", GeometricScaling)
    register_architecture(ArchitectureEntry("Toy2ForCausalLM", ToyConfig, build_toy, model_types=("toy2",)))
    try:
        write_random_model({"architectures": ["Toy2ForCausalLM"], "model_type": "toy2", "vocab_size": 40}, tmp_path, seed=5)
        model = load_model(tmp_path, dtype="float32")
        runner = make_runner(model, page_size=4, max_tokens=96, max_requests=3)
        reqs = {"a": torch.randint(0, 40, (29,)).tolist(), "b": torch.randint(0, 40, (10,)).tolist()}
        with torch.inference_mode():
            whole = {k: runner.step([StepEntry(k + "w", v, list(range(len(v))))]).cpu() for k, v in reqs.items()}
            runner.end(["aw", "bw"])
            got = {"a": [], "b": []}
            got["a"].append(runner.step([StepEntry("a", reqs["a"][:7], list(range(7)))]).cpu())
            mixed = runner.step([StepEntry("b", reqs["b"][:9], list(range(9))), StepEntry("a", reqs["a"][7:8], [0])]).cpu()
            got["b"].append(mixed[:9]), got["a"].append(mixed[9:])
            mixed = runner.step([StepEntry("a", reqs["a"][8:], list(range(21))), StepEntry("b", reqs["b"][9:], [0])]).cpu()
            got["a"].append(mixed[:21]), got["b"].append(mixed[21:])
            runner.end(["a", "b"])
        for k in reqs:
            assert torch.allclose(torch.cat(got[k]), whole[k], atol=2e-5, rtol=1e-4)
        _, w = plain_llama.read_model_folder(tmp_path)

        def attention(x, p, g):
            n, T = plain_llama.rms_norm(x, w[p + "n1.weight"], 1e-5), x.shape[0]
            q = (n @ w[p + "attn.q_proj.weight"].T).view(T, HEADS, D).transpose(0, 1) * g[None, :, None]
            k = (n @ w[p + "attn.k_proj.weight"].T).view(T, KV, D).transpose(0, 1) / g[None, :, None]
            v = (n @ w[p + "attn.v_proj.weight"].T).view(T, KV, D).transpose(0, 1)
            return x + plain_llama.causal_attention(q, k, v, HEADS // KV).transpose(0, 1).reshape(T, HEADS * D) @ w[p + "attn.o_proj.weight"].T

        x = w["emb.weight"][torch.tensor(reqs["a"])]
        T = x.shape[0]
        x = attention(x, "l0.", torch.pow(torch.tensor(BASE, dtype=torch.float64), torch.arange(T, dtype=torch.float64)))
        n = plain_llama.rms_norm(x, w["l0.n2.weight"], 1e-5)
        prob = torch.softmax(n @ w["l0.moe.router.weight"].T, dim=-1)
        weight, choice = prob.max(dim=-1)
        assert len(set(choice.tolist())) > 1                       # the tokens really go to different experts
        routed = torch.stack([(torch.relu(n[t] @ w[f"l0.moe.experts.{int(choice[t])}.up.weight"].T)
                               @ w[f"l0.moe.experts.{int(choice[t])}.down.weight"].T) * weight[t] for t in range(T)])
        x = x + routed
        x = attention(x, "l1.", torch.ones(T, dtype=torch.float64))
        x = x + plain_llama.swiglu_mlp(plain_llama.rms_norm(x, w["l1.n2.weight"], 1e-5), w["l1.ffn.gate_proj.weight"],
                                       w["l1.ffn.up_proj.weight"], w["l1.ffn.down_proj.weight"])
        want = plain_llama.rms_norm(x, w["final.weight"], 1e-5) @ w["head.weight"].T
        assert torch.allclose(whole["a"].double(), want, atol=5e-5, rtol=2e-4), (whole["a"].double() - want).abs().max()
    finally:
        unregister_part("feed_forward", "toy_routed")
        unregister_part("position", "geometric")
        unregister_architecture("Toy2ForCausalLM")


def test_a_toy_mixer_with_keys_narrower_than_values_and_a_stage_after_the_embedding(tmp_path):
    """Two more parts defined here.  A mixer that caches a key of 8 and a value of 24 elements per token (the
    cache manager gives it pages that hold keys and values of different widths, as views) and reads them back
    through the block table; it walks the step's entries on the host, so it declares itself not capturable and
    the model's decode steps run uncaptured.  And a stage between the embedding and the first block that adds a
    learned absolute position table and multiplies by a constant.  Registered, given random weights, loaded and
    stepped whole, in portions and token by token, against plain arithmetic; nothing of the package is edited."""
    need_gpu()
    from torchinferno_b200.config.registry import ArchitectureEntry, register_architecture, unregister_architecture
    from torchinferno_b200.engine.batch import StepEntry
    from torchinferno_b200.engine.factory import load_model, make_runner
    from torchinferno_b200.models.spec import BlockSpec, LayerCall, ModelSpec
    from torchinferno_b200.parts.base import (CacheSpec, Mixer, PartSpec, StreamStage, WeightSpec, register_part,
                                              unregister_part)
    from torchinferno_b200.weights.random_init import write_random_model
    WIDTH, KEY, POSITIONS, SCALE = 24, 8, 64, 1.7

    class WideValueMixer(Mixer):
        capturable = False                                           # (it reads ctx.batch.entries on the host)

        def __init__(self, *, width, key_dim, dtype, device):
            super().__init__(dtype=dtype, device=device)
            self.width, self.key_dim = width, key_dim

        def weight_specs(self):
            return [WeightSpec("q.weight", (self.key_dim, self.width), std=0.4), WeightSpec("k.weight", (self.key_dim, self.width), std=0.4),
                    WeightSpec("o.weight", (self.width, self.width), std=0.2)]

        def bind(self, weights):
            self.wq, self.wk, self.wo = (weights[n].float() for n in ("q.weight", "k.weight", "o.weight"))

        def cache_spec(self):
            return CacheSpec(1, self.key_dim, value_dim=self.width)

        def forward(self, x, ctx):
            kv, page = ctx.kv, ctx.kv.page_size
            assert kv.keys.shape[1:] == (1, page, self.key_dim) and kv.values.shape[1:] == (1, page, self.width)
            out = torch.empty_like(x)
            for e in ctx.batch.entries:
                rows = x[e.q_start:e.q_start + e.q_len].float()
                positions = torch.arange(e.kv_start, e.kv_start + e.q_len, device=x.device)
                table = kv.block_table[e.slot]
                pages, offsets = table[positions // page].long(), positions % page
                kv.keys[pages, 0, offsets] = (rows @ self.wk.T).to(kv.keys.dtype)
                kv.values[pages, 0, offsets] = rows.to(kv.values.dtype)
                every = torch.arange(0, e.kv_start + e.q_len, device=x.device)
                keys = kv.keys[table[every // page].long(), 0, every % page].float()
                values = kv.values[table[every // page].long(), 0, every % page].float()
                scores = (rows @ self.wq.T) @ keys.T / self.key_dim ** 0.5
                scores = scores.masked_fill(every[None, :] > positions[:, None], float("-inf"))
                out[e.q_start:e.q_start + e.q_len] = ((torch.softmax(scores, -1) @ values) @ self.wo.T).to(x.dtype)
            return out

    class LearnedPositions(StreamStage):
        def __init__(self, *, width, positions, scale, dtype, device):
            super().__init__(dtype=dtype, device=device)
            self.width, self.positions, self.scale = width, positions, scale

        def weight_specs(self):
            return [WeightSpec("table.weight", (self.positions, self.width), std=0.3)]

        def bind(self, weights):
            self.table = weights["table.weight"].float()

        def forward(self, stream, ctx):
            stream.residual.add_(self.table[ctx.batch.positions.long()]).mul_(self.scale)

    @dataclasses.dataclass(frozen=True)
    class Toy3Config:
        vocab_size: int

        @classmethod
        def from_dict(cls, data):
            return cls(data["vocab_size"])

    def build_toy3(cfg):
        norm = PartSpec("rmsnorm", {"width": WIDTH, "eps": 1e-5})
        block = PartSpec("prenorm", {
            "mixer": PartSpec("wide_value", {"width": WIDTH, "key_dim": KEY}, prefix="mix."),
            "feed_forward": PartSpec("swiglu", {"hidden_size": WIDTH, "intermediate_size": 40}, prefix="ffn."),
            "mixer_norm": dataclasses.replace(norm, prefix="n1."), "feed_forward_norm": dataclasses.replace(norm, prefix="n2.")})
        return ModelSpec(architecture="Toy3ForCausalLM", hidden_size=WIDTH, vocab_size=cfg.vocab_size, max_positions=POSITIONS,
                         embedding_name="emb.weight", layers=(BlockSpec(block, "l0."), BlockSpec(block, "l1.")),
                         schedule=(LayerCall(0, 0), LayerCall(1, 1)), final_norm=dataclasses.replace(norm, prefix="final."),
                         head_name="head.weight",
                         after_embedding=PartSpec("learned_positions", {"width": WIDTH, "positions": POSITIONS, "scale": SCALE}, prefix="pos."))

    register_part("mixer", "wide_value", WideValueMixer)
    register_part("stream_stage", "learned_positions", LearnedPositions)
    register_architecture(ArchitectureEntry("Toy3ForCausalLM", Toy3Config, build_toy3, model_types=("toy3",)))
    try:
        write_random_model({"architectures": ["Toy3ForCausalLM"], "model_type": "toy3", "vocab_size": 40}, tmp_path, seed=3)
        model = load_model(tmp_path, dtype="float32")
        assert not model.capturable() and [c.value_width for c in model.cache_requirements()] == [WIDTH, WIDTH]
        runner = make_runner(model, page_size=4, max_tokens=96, max_requests=2)
        assert runner.cache.groups[0].pool.shape == (2, 24, 4 * (KEY + WIDTH)) and not runner._graph_ok
        tokens = torch.randint(0, 40, (29,)).tolist()
        with torch.inference_mode():
            whole = runner.step([StepEntry("w", tokens, list(range(29)))]).cpu()
            runner.end(["w"])
            cut = [runner.step([StepEntry("c", tokens[:7], list(range(7)))]).cpu(),
                   runner.step([StepEntry("c", tokens[7:20], list(range(13)))]).cpu()]
            cut += [runner.step([StepEntry("c", [t], [0])]).cpu() for t in tokens[20:]]          # single tokens, uncaptured
            runner.end(["c"])
        assert runner.graph_replays == 0 and runner.cache.free_pages() == [24]
        assert torch.allclose(torch.cat(cut), whole, atol=1e-5, rtol=1e-4)
        _, w = plain_llama.read_model_folder(tmp_path)
        T = len(tokens)
        x = (w["emb.weight"][torch.tensor(tokens)] + w["pos.table.weight"][:T]) * SCALE
        for p in ("l0.", "l1."):
            n = plain_llama.rms_norm(x, w[p + "n1.weight"], 1e-5)
            scores = (n @ w[p + "mix.q.weight"].T) @ (n @ w[p + "mix.k.weight"].T).T / KEY ** 0.5
            scores = scores.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
            x = x + (torch.softmax(scores, -1) @ n) @ w[p + "mix.o.weight"].T
            x = x + plain_llama.swiglu_mlp(plain_llama.rms_norm(x, w[p + "n2.weight"], 1e-5), w[p + "ffn.gate_proj.weight"],
                                           w[p + "ffn.up_proj.weight"], w[p + "ffn.down_proj.weight"])
        want = plain_llama.rms_norm(x, w["final.weight"], 1e-5) @ w["head.weight"].T
        assert torch.allclose(whole.double(), want, atol=5e-5, rtol=2e-4), (whole.double() - want).abs().max()
    finally:
        unregister_part("mixer", "wide_value")
        unregister_part("stream_stage", "learned_positions")
        unregister_architecture("Toy3ForCausalLM")


def test_a_toy_norm_and_a_toy_arrangement_of_a_block_are_registered_and_stepped(tmp_path):
    """The two kinds of part the other toy tests leave alone, defined here and unknown to the framework: a norm with
    a mean and a bias (y = (x - mean) / sqrt(var + eps) * w + b, its own way of folding the pending delta in), and a
    block that arranges its parts differently: one norm, whose rows go to the mixer and to the feed-forward side by
    side, and one add (h = h + mixer(n(h)) + feed_forward(n(h))).  The first layer is such a block, the second the
    framework's pre-norm block with the toy norm in both places.  Stepped whole, in portions and mixed, against plain
    arithmetic."""
    need_gpu()
    from torchinferno_b200.config.registry import ArchitectureEntry, register_architecture, unregister_architecture
    from torchinferno_b200.engine.batch import StepEntry
    from torchinferno_b200.engine.factory import load_model, make_runner
    from torchinferno_b200.models.spec import BlockSpec, LayerCall, ModelSpec
    from torchinferno_b200.parts.base import Block, Norm, PartSpec, WeightSpec, build_part, register_part, unregister_part
    from torchinferno_b200.weights.random_init import write_random_model
    WIDTH, INTER, HEADS, KV, D, EPS = 40, 24, 4, 2, 16, 1e-4

    class CenteredNorm(Norm):
        def __init__(self, *, width, eps, dtype, device):
            super().__init__(dtype=dtype, device=device)
            self.width, self.eps = width, eps

        def weight_specs(self):
            return [WeightSpec("weight", (self.width,), init="normal", std=0.5, role="vector"),
                    WeightSpec("bias", (self.width,), init="normal", std=0.3, role="vector")]

        def bind(self, weights):
            self.weight, self.bias = weights["weight"].float(), weights["bias"].float()

        def forward(self, residual, out, rows=None):
            x = residual if rows is None else residual[rows.long()]
            centred = x - x.mean(-1, keepdim=True)
            out.copy_((centred * torch.rsqrt(centred.square().mean(-1, keepdim=True) + self.eps) * self.weight + self.bias).to(out.dtype))
            return out

        def add_forward(self, delta, residual, out, rows=None):
            if rows is None:
                residual += delta.float()                       # the stream takes the delta for good
                return self.forward(residual, out)
            chosen = rows.long()                                # only looked at: the stream keeps the delta pending
            return self.forward((residual[chosen] + delta[chosen].float()).contiguous(), out)

    class SideBySideBlock(Block):
        def __init__(self, *, mixer, feed_forward, norm, dtype, device):
            super().__init__(dtype=dtype, device=device)
            as_spec = lambda v: v if isinstance(v, PartSpec) else PartSpec(**v)
            self.specs = {"mixer": as_spec(mixer), "feed_forward": as_spec(feed_forward), "norm": as_spec(norm)}
            self.mixer = build_part("mixer", self.specs["mixer"], dtype=dtype, device=device)
            self.feed_forward = build_part("feed_forward", self.specs["feed_forward"], dtype=dtype, device=device)
            self.norm = build_part("norm", self.specs["norm"], dtype=dtype, device=device)

        def named_parts(self):
            return [(self.specs[k].prefix, getattr(self, k)) for k in ("norm", "mixer", "feed_forward")]

        def forward(self, stream, ctx):
            rows = stream.normed(self.norm)
            stream.add(self.mixer.forward(rows, ctx) + self.feed_forward.forward(rows, ctx))

    @dataclasses.dataclass(frozen=True)
    class ToyConfig:
        vocab_size: int

        @classmethod
        def from_dict(cls, data):
            return cls(data["vocab_size"])

    def build_toy(cfg):
        norm = PartSpec("centred", {"width": WIDTH, "eps": EPS})
        attention = PartSpec("gqa_attention", {"hidden_size": WIDTH, "heads": HEADS, "kv_heads": KV, "head_dim": D,
                                               "position": PartSpec("rotary", {"head_dim": D, "theta": 100.0})}, prefix="attn.")
        ffn = PartSpec("swiglu", {"hidden_size": WIDTH, "intermediate_size": INTER}, prefix="ffn.")
        side = PartSpec("side_by_side", {"mixer": attention, "feed_forward": ffn, "norm": dataclasses.replace(norm, prefix="n.")})
        pre = PartSpec("prenorm", {"mixer": attention, "feed_forward": ffn, "mixer_norm": dataclasses.replace(norm, prefix="n1."),
                                   "feed_forward_norm": dataclasses.replace(norm, prefix="n2.")})
        return ModelSpec(architecture="Toy4ForCausalLM", hidden_size=WIDTH, vocab_size=cfg.vocab_size, max_positions=128,
                         embedding_name="emb.weight", layers=(BlockSpec(side, "l0."), BlockSpec(pre, "l1.")),
                         schedule=(LayerCall(0, 0), LayerCall(1, 1)),
                         final_norm=dataclasses.replace(norm, prefix="final."), head_name="head.weight")

    register_part("norm", "centred", CenteredNorm)
    register_part("block", "side_by_side", SideBySideBlock)
    register_architecture(ArchitectureEntry("Toy4ForCausalLM", ToyConfig, build_toy, model_types=("toy4",)))
    try:
        write_random_model({"architectures": ["Toy4ForCausalLM"], "model_type": "toy4", "vocab_size": 50}, tmp_path, seed=8)
        model = load_model(tmp_path, dtype="float32")
        runner = make_runner(model, page_size=4, max_tokens=96, max_requests=3)
        reqs = {"a": torch.randint(0, 50, (27,)).tolist(), "b": torch.randint(0, 50, (11,)).tolist()}
        with torch.inference_mode():
            whole = {k: runner.step([StepEntry(k + "w", v, list(range(len(v))))]).cpu() for k, v in reqs.items()}
            runner.end(["aw", "bw"])
            got = {"a": [], "b": []}
            got["a"].append(runner.step([StepEntry("a", reqs["a"][:5], list(range(5)))]).cpu())
            mixed = runner.step([StepEntry("b", reqs["b"][:10], list(range(10))), StepEntry("a", reqs["a"][5:6], [0])]).cpu()
            got["b"].append(mixed[:10]), got["a"].append(mixed[10:])
            mixed = runner.step([StepEntry("a", reqs["a"][6:], [0, 20]), StepEntry("b", reqs["b"][10:], [0])]).cpu()   # wanted rows only
            runner.end(["a", "b"])
        assert torch.allclose(torch.cat(got["a"]), whole["a"][:6], atol=2e-5, rtol=1e-4)
        assert torch.allclose(mixed[:2], whole["a"][[6, 26]], atol=2e-5, rtol=1e-4)
        assert torch.allclose(torch.cat([got["b"][0], mixed[2:]]), whole["b"], atol=2e-5, rtol=1e-4)
        _, w = plain_llama.read_model_folder(tmp_path)

        def norm(x, p):
            centred = x - x.mean(-1, keepdim=True)
            return centred * torch.rsqrt(centred.square().mean(-1, keepdim=True) + EPS) * w[p + "weight"] + w[p + "bias"]

        def attention(n, p):
            T = n.shape[0]
            inv_freq = 1.0 / (100.0 ** (torch.arange(0, D, 2, dtype=torch.float64) / D))
            q = (n @ w[p + "attn.q_proj.weight"].T).view(T, HEADS, D).transpose(0, 1)
            k = (n @ w[p + "attn.k_proj.weight"].T).view(T, KV, D).transpose(0, 1)
            v = (n @ w[p + "attn.v_proj.weight"].T).view(T, KV, D).transpose(0, 1)
            q, k = plain_llama.rotary(q, torch.arange(T), inv_freq), plain_llama.rotary(k, torch.arange(T), inv_freq)
            return plain_llama.causal_attention(q, k, v, HEADS // KV).transpose(0, 1).reshape(T, HEADS * D) @ w[p + "attn.o_proj.weight"].T

        def ffn(n, p):
            return plain_llama.swiglu_mlp(n, w[p + "ffn.gate_proj.weight"], w[p + "ffn.up_proj.weight"], w[p + "ffn.down_proj.weight"])

        x = w["emb.weight"][torch.tensor(reqs["a"])]
        n = norm(x, "l0.n.")
        x = x + attention(n, "l0.") + ffn(n, "l0.")
        x = x + attention(norm(x, "l1.n1."), "l1.")
        x = x + ffn(norm(x, "l1.n2."), "l1.")
        want = norm(x, "final.") @ w["head.weight"].T
        assert torch.allclose(whole["a"].double(), want, atol=5e-5, rtol=2e-4), (whole["a"].double() - want).abs().max()
    finally:
        unregister_part("norm", "centred")
        unregister_part("block", "side_by_side")
        unregister_architecture("Toy4ForCausalLM")


@pytest.mark.parametrize("name", ["D", "E"])
def test_the_native_block_call_gives_the_bits_of_the_part_by_part_sequence(model_folders, name, monkeypatch):
    """A block of the built-in parts in bfloat16 is issued as one call into the CUDA library; it must launch the
    same kernels with the same choices as the parts do one by one: logits equal bit for bit, for a whole prompt,
    portions, a mixed step and decoding (captured and not)."""
    need_gpu()
    from torchinferno_b200.engine.batch import StepEntry
    from torchinferno_b200.engine.factory import load_model, make_runner
    from torchinferno_b200.parts import block as block_module
    cfg = json.loads((model_folders[name] / "config.json").read_text())
    g = torch.Generator().manual_seed(3)
    a, b = (torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in (150, 41))

    def run(native, graphs):
        monkeypatch.setattr(block_module, "NATIVE_BLOCKS", native)
        model = load_model(model_folders[name], dtype="bfloat16")
        runner = make_runner(model, page_size=16, max_tokens=512, max_requests=4)
        runner.use_cuda_graphs = graphs
        outs = []
        with torch.inference_mode():
            # (a captured step returns the graph's own output buffer: read it before the next step)
            outs.append(runner.step([StepEntry("a", a[:100], [0, 99])]).cpu())
            outs.append(runner.step([StepEntry("a", a[100:101], [0]), StepEntry("b", b[:40], [3, 39])]).cpu())
            for t in range(101, 106):
                outs.append(runner.step([StepEntry("a", a[t:t + 1], [0]), StepEntry("b", [b[40]] if t == 101 else [7], [0])]).cpu())
        used = [blk._native is not None and blk._native is not block_module._UNKNOWN for blk in model.blocks]
        return torch.cat(outs), used

    parts, used_parts = run(False, False)
    for graphs in (False, True):
        native, used_native = run(True, graphs)
        assert all(used_native) and not any(used_parts)
        assert torch.equal(native, parts), ((native - parts).abs().max(), (native != parts).any(dim=1).tolist())
