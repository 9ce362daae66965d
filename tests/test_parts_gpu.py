"""Each part alone against its plain formula, the layer order as data (a layer named
twice, a layer that reads another layer's cache), and a toy mixer with state of its
own that is defined here, registered from here and stepped through the engine
without any change to the package."""

import json
import math
import os
import tempfile

import numpy as np
import pytest
import torch

import plain_llama as P

pytestmark = pytest.mark.gpu

DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 3e-5, "bfloat16": 3e-2}


def _ctx(dtype, max_positions=256):
    from kv_cache_optimization_for_llm_b200.parts import BuildContext
    dev = torch.device("cuda:0")
    return BuildContext(dtype=DT[dtype], device=dev, max_positions=max_positions,
                        status=torch.zeros(1, dtype=torch.int32, device=dev))


def _w(rng, shape, dtype, std=0.1):
    """Random weights that are exactly representable in the compute dtype."""
    t = torch.as_tensor(rng.normal(size=shape) * std).to(DT[dtype])
    return t.cuda(), t.float().numpy().astype(np.float64)


def _rel(got, ref):
    return np.abs(got.detach().float().cpu().numpy().astype(np.float64) - ref).max() / np.abs(ref).max()


class _Manager:
    """Stands in for the cache manager when a part is run alone: one request, pages 0..n."""
    def __init__(self, n_pages):
        self.table = list(range(n_pages))

    def slot_of(self, rid):
        return 0

    def block_table(self, rid, g):
        return self.table


def _batch(ctx, tokens, start, page_size, max_pages):
    from kv_cache_optimization_for_llm_b200.engine.batch import BatchBuilder, StepEntry
    b = BatchBuilder(512, 4, [max_pages], ctx.device, ctx.status)
    n_pages = -(-(start + len(tokens)) // page_size)
    return b.build([StepEntry(0, tokens, start, list(range(len(tokens))))], _Manager(n_pages))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_norm_embedding_head_feed_forward_alone(dtype):
    from kv_cache_optimization_for_llm_b200.parts import lookup
    rng = np.random.default_rng(0)
    ctx = _ctx(dtype)
    H, I, V, T = 120, 200, 333, 9
    # norm
    wn = torch.as_tensor(1 + 0.1 * rng.normal(size=H), dtype=torch.float32).cuda()
    norm = lookup("norm", "rmsnorm")({"size": H, "eps": 2e-5}, {"weight": wn}, ctx)
    resid = torch.as_tensor(rng.normal(size=(T, H)), dtype=torch.float32).cuda()
    r0 = resid.cpu().numpy().astype(np.float64)
    assert _rel(norm.forward(resid), P.rms_norm(r0, wn.cpu().numpy().astype(np.float64), 2e-5)) < TOL[dtype]
    # embedding and head share one table when tied
    tab, tab64 = _w(rng, (V, H), dtype, 1.0)
    emb = lookup("embedding", "token_embedding")({"vocab_size": V, "hidden_size": H}, {"table": tab}, ctx)
    toks = [0, V - 1, 17, 17, 200, 3, 4, 5, 6]
    batch = _batch(ctx, toks, 0, 16, 4)
    assert np.array_equal(emb.forward(batch).cpu().numpy().astype(np.float64), tab64[toks])
    head = lookup("head", "linear_head")({"vocab_size": V, "hidden_size": H}, {"weight": tab}, ctx)
    x, x64 = _w(rng, (T, H), dtype, 1.0)
    out = head.forward(x)
    assert out.dtype == torch.float32 and _rel(out, x64 @ tab64.T) < TOL[dtype]
    # feed-forward
    wg, wg64 = _w(rng, (I, H), dtype)
    wu, wu64 = _w(rng, (I, H), dtype)
    wd, wd64 = _w(rng, (H, I), dtype)
    ff = lookup("feed_forward", "swiglu")({"hidden_size": H, "intermediate_size": I},
                                          {"gate": wg, "up": wu, "down": wd}, ctx)
    ref = P.swiglu_part(x64, {"gate_proj.weight": wg64, "up_proj.weight": wu64, "down_proj.weight": wd64}, "")
    assert _rel(ff.forward(x, batch), ref) < TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nq,nkv,d,window,scaling", [
    (4, 2, 16, None, None), (6, 3, 32, 7, {"factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                                           "original_max_position_embeddings": 32}),
    (3, 1, 64, None, {"factor": 2.0, "low_freq_factor": 1.0, "high_freq_factor": 3.0,
                      "original_max_position_embeddings": 16})])
def test_attention_mixer_alone_in_portions(dtype, nq, nkv, d, window, scaling):
    """The attention part with its rotary encoding, fed a sequence in three portions
    (so that it reads its own cache), against the plain whole-sequence formula."""
    from kv_cache_optimization_for_llm_b200.cache.specs import PagedKVBinding, PagedKVSpec
    from kv_cache_optimization_for_llm_b200.models.spec import PartSpec
    from kv_cache_optimization_for_llm_b200.parts import lookup
    rng = np.random.default_rng(d)
    ctx = _ctx(dtype)
    H, T, page = 72, 45, 8
    w, w64 = {}, {}
    for role, shape in (("q", (nq * d, H)), ("k", (nkv * d, H)), ("v", (nkv * d, H)), ("o", (H, nq * d))):
        w[role], w64[f"{role}_proj.weight"] = _w(rng, shape, dtype, 0.3)
    rope = PartSpec("rope", {"head_dim": d, "rotary_dim": d, "theta": 10000.0, "scaling": scaling})
    attn = lookup("mixer", "attention")({"hidden_size": H, "num_heads": nq, "num_kv_heads": nkv, "head_dim": d,
                                         "window": window, "position": rope}, w, ctx)
    assert attn.cache_spec() == PagedKVSpec(nkv, d, window)
    x, x64 = _w(rng, (T, H), dtype, 1.0)
    cfg = {"num_attention_heads": nq, "num_key_value_heads": nkv, "head_dim": d, "hidden_size": H}
    inv = P.rope_inv_freq(d, 10000.0, scaling)
    ref = P.gqa_attention_part(x64, w64, "", cfg, np.arange(T), inv, window=window)
    n_pages = -(-T // page)
    kv = torch.zeros((2, n_pages + 1, nkv, page, d), dtype=DT[dtype], device="cuda")
    binding = PagedKVBinding(k=kv[0], v=kv[1], group=0, page_size=page)
    outs = []
    for a, b in ((0, 20), (20, 22), (22, 45)):
        batch = _batch(ctx, [0] * (b - a), a, page, n_pages + 1)
        outs.append(attn.forward(x[a:b].contiguous(), batch, binding))
    assert int(ctx.status.item()) == 0
    assert _rel(torch.cat(outs), ref) < TOL[dtype]


# ---------------------------------------------------------------------------------
# A toy architecture, defined and registered here: layers of two kinds (attention and
# a mixer with a fixed-size state per request), a layer that runs twice, and a layer
# that reads another layer's cache.
# ---------------------------------------------------------------------------------

def _register_toy():
    from kv_cache_optimization_for_llm_b200.cache.specs import SlotStateSpec
    from kv_cache_optimization_for_llm_b200.models.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
    from kv_cache_optimization_for_llm_b200.parts import Part, register
    from kv_cache_optimization_for_llm_b200.registry import register_architecture
    from kv_cache_optimization_for_llm_b200.weights.loader import WeightSpec

    @register("mixer", "toy_decay")
    class DecayMixer(Part):
        """s_t = decay * s_{t-1} + x_t per request, y_t = s_t . W^T.  The state s lives in
        the request's slot between steps.  Torch ops: a toy, not a product kernel."""

        @classmethod
        def weight_specs(cls, params):
            return {"w": WeightSpec((params["hidden_size"], params["hidden_size"]))}

        def __init__(self, params, weights, ctx):
            super().__init__(params, weights, ctx)
            self.decay, self.w, self.h = float(params["decay"]), weights["w"], int(params["hidden_size"])

        def cache_spec(self):
            return SlotStateSpec((self.h,), torch.float32)

        def forward(self, x, batch, cache):
            out = torch.empty_like(x)
            qs, starts = batch.host["q_start"], batch.host["req_start"]
            slots = batch.slots.tolist()
            for r in range(batch.num_reqs):
                s = cache.state[slots[r]]
                if starts[r] == 0:
                    s.zero_()                      # a request that starts over starts from nothing
                for t in range(int(qs[r]), int(qs[r + 1])):
                    s.mul_(self.decay).add_(x[t].float())
                    out[t] = (s.to(x.dtype) @ self.w.t())
            return out

    def build(cfg):
        H, V = cfg["hidden_size"], cfg["vocab_size"]
        norm = lambda name: PartSpec("rmsnorm", {"size": H, "eps": cfg["eps"]}, {"weight": name})
        ff = lambda p: PartSpec("swiglu", {"hidden_size": H, "intermediate_size": cfg["inter"]},
                                {"gate": p + "ff.gate", "up": p + "ff.up", "down": p + "ff.down"})
        rope = PartSpec("rope", {"head_dim": cfg["head_dim"], "rotary_dim": cfg["head_dim"], "theta": 1000.0, "scaling": None})
        def attn(p, window):
            return PartSpec("attention", {"hidden_size": H, "num_heads": cfg["heads"], "num_kv_heads": cfg["kv_heads"],
                                          "head_dim": cfg["head_dim"], "window": window, "position": rope},
                            {r: f"{p}attn.{r}" for r in "qkvo"})
        layers = []
        windows = cfg.get("windows") or [None] * len(cfg["mixers"])
        for i, kind in enumerate(cfg["mixers"]):
            p = f"l{i}."
            mixer = attn(p, windows[i]) if kind == "attention" else PartSpec("toy_decay", {"hidden_size": H, "decay": cfg["decay"]}, {"w": p + "decay.w"})
            layers.append(LayerSpec("prenorm", dict(mixer=mixer, mixer_norm=norm(p + "n1"), feed_forward=ff(p),
                                                    ff_norm=norm(p + "n2"))))
        return ModelSpec(architecture="ToyForCausalLM", hidden_size=H, vocab_size=V, max_position=cfg["max_pos"],
                         embedding=PartSpec("token_embedding", {"vocab_size": V, "hidden_size": H}, {"table": "emb"}),
                         layers=layers,
                         schedule=[ScheduleEntry(l, c) for l, c in cfg["schedule"]],
                         final_norm=norm("nf"),
                         lm_head=PartSpec("linear_head", {"vocab_size": V, "hidden_size": H}, {"weight": "emb"}))

    register_architecture("ToyForCausalLM", lambda d: d, build)


TOY = {"architectures": ["ToyForCausalLM"], "hidden_size": 48, "vocab_size": 97, "inter": 80, "eps": 1e-5,
       "heads": 4, "kv_heads": 2, "head_dim": 16, "max_pos": 96, "decay": 0.8,
       # layer 0: attention; layer 1: decay mixer; layer 2: attention.
       # schedule: 0, 1, 2 reading 0's cache, 1 again (with a state of its own), 0 again (with pages of its own)
       "mixers": ["attention", "toy_decay", "attention"],
       "schedule": [[0, None], [1, None], [2, 0], [1, None], [0, None]]}


def _toy_plain(cfg, w, tokens):
    """The toy model, whole sequence, no cache, numpy."""
    T, H, d = len(tokens), cfg["hidden_size"], cfg["head_dim"]
    nq, nkv = cfg["heads"], cfg["kv_heads"]
    inv = P.rope_inv_freq(d, 1000.0)
    cos, sin = P.rope_tables(np.arange(T), inv)
    h = w["emb"][np.asarray(tokens)]
    kv_of = {}
    windows = cfg.get("windows") or [None] * len(cfg["mixers"])
    for idx, (l, cache_of) in enumerate(cfg["schedule"]):
        p = f"l{l}."
        x = P.rms_norm(h, w[p + "n1"], cfg["eps"])
        if cfg["mixers"][l] == "attention":
            q = P.apply_rope(P.linear(x, w[p + "attn.q"]).reshape(T, nq, d), cos, sin)
            if cache_of is None:
                k = P.apply_rope(P.linear(x, w[p + "attn.k"]).reshape(T, nkv, d), cos, sin)
                v = P.linear(x, w[p + "attn.v"]).reshape(T, nkv, d)
                kv_of[idx] = (k, v)
            else:
                k, v = kv_of[cache_of]
            a = P.linear(P.attention(q, k, v, window=windows[l]).reshape(T, nq * d), w[p + "attn.o"])
        else:
            s = np.zeros(H)
            a = np.zeros((T, H))
            for t in range(T):
                s = cfg["decay"] * s + x[t]
                a[t] = w[p + "decay.w"] @ s
        h = h + a
        x = P.rms_norm(h, w[p + "n2"], cfg["eps"])
        h = h + P.swiglu_part(x, {"gate_proj.weight": w[p + "ff.gate"], "up_proj.weight": w[p + "ff.up"],
                                  "down_proj.weight": w[p + "ff.down"]}, "")
    return P.linear(P.rms_norm(h, w["nf"], cfg["eps"]), w["emb"])


def test_toy_architecture_with_a_state_mixer_registers_builds_and_steps():
    from kv_cache_optimization_for_llm_b200 import EngineConfig
    from kv_cache_optimization_for_llm_b200.engine.batch import StepEntry
    from kv_cache_optimization_for_llm_b200.engine.runner import ModelRunner
    from kv_cache_optimization_for_llm_b200.registry import known_architectures
    from kv_cache_optimization_for_llm_b200.weights import write_random_model
    _register_toy()
    assert "ToyForCausalLM" in known_architectures()
    d = tempfile.mkdtemp(prefix="kvb200_toy_")
    write_random_model(d, TOY, seed=5, std=0.2)
    w = P.read_safetensors(os.path.join(d, "model.safetensors"))
    assert "l1.decay.w" in w and "l2.attn.q" in w and "l2.attn.k" in w
    r = ModelRunner(d, EngineConfig(dtype="float32", page_size=4, num_pages=40, max_num_seqs=3,
                                    max_num_batched_tokens=64, max_model_len=96, use_cuda_graphs=False))
    # two paged entries with pages of their own (schedule entries 0 and 4), two states (1 and 3)
    assert r.cache.group_entries == [2] and sorted(r.cache.states) == [1, 3]
    rng = np.random.default_rng(2)
    seqs = [rng.integers(0, 97, n).tolist() for n in (23, 40)]
    refs = [_toy_plain(TOY, w, s) for s in seqs]
    # request 0 whole; request 1 in portions beside request 0's decode-like single tokens
    got0 = r.step([StepEntry(0, seqs[0][:15], 0, range(15))]).cpu().numpy()
    assert np.abs(got0 - refs[0][:15]).max() / np.abs(refs[0]).max() < 3e-5
    pos0, pos1 = 15, 0
    for n1 in (7, 2, 1, 13, 5, 1, 1, 10):
        entries = [StepEntry(1, seqs[1][pos1:pos1 + n1], pos1, range(n1))]
        expect = [refs[1][pos1:pos1 + n1]]
        if pos0 < len(seqs[0]):
            entries.append(StepEntry(0, [seqs[0][pos0]], pos0, [0]))
            expect.append(refs[0][pos0:pos0 + 1])
            pos0 += 1
        got = r.step(entries).cpu().numpy()
        ref = np.concatenate(expect)
        assert np.abs(got - ref).max() / np.abs(ref).max() < 3e-5, (pos0, pos1)
        pos1 += n1
    assert pos1 == 40
    r.check_status()
    # a request that is released and starts again in the same slot starts from a clean state
    r.release(1)
    got = r.step([StepEntry(2, seqs[1][:9], 0, range(9))]).cpu().numpy()
    assert np.abs(got - refs[1][:9]).max() / np.abs(refs[1]).max() < 3e-5
    assert r.manager.check() == ""


TOY_WINDOWED = {"architectures": ["ToyForCausalLM"], "hidden_size": 48, "vocab_size": 97, "inter": 80, "eps": 1e-5,
                "heads": 4, "kv_heads": 2, "head_dim": 16, "max_pos": 96, "decay": 0.8,
                # a layer that reads only its newest 9 keys beside a layer that reads them all:
                # two cache groups, each with pages and block tables of its own
                "mixers": ["attention", "attention", "attention"], "windows": [9, None, 9],
                "schedule": [[0, None], [1, None], [2, None]]}


def test_windowed_and_full_layers_have_page_groups_of_their_own():
    """A model whose layers differ in what they keep: the window group gives pages back as
    the window passes them while the full group keeps all; logits stay right through
    portions, single tokens and the window's edge, in a pool far smaller than the sequence
    for the window group."""
    from kv_cache_optimization_for_llm_b200 import EngineConfig
    from kv_cache_optimization_for_llm_b200.engine.batch import StepEntry
    from kv_cache_optimization_for_llm_b200.engine.runner import ModelRunner
    from kv_cache_optimization_for_llm_b200.weights import write_random_model
    _register_toy()
    d = tempfile.mkdtemp(prefix="kvb200_toyw_")
    write_random_model(d, TOY_WINDOWED, seed=6, std=0.2)
    w = P.read_safetensors(os.path.join(d, "model.safetensors"))
    for dtype, tol in (("float32", 3e-5), ("bfloat16", 4e-2)):
        r = ModelRunner(d, EngineConfig(dtype=dtype, page_size=4, num_pages=24, max_num_seqs=2,
                                        max_num_batched_tokens=64, max_model_len=96, use_cuda_graphs=False))
        m = r.manager
        assert m.num_groups() == 2
        groups = {m.group(g).window: g for g in range(2)}
        gw, gf = groups[9], groups[0]
        assert r.cache.group_entries[gw] == 2 and r.cache.group_entries[gf] == 1
        seq = np.random.default_rng(8).integers(0, 97, 90).tolist()
        ref = _toy_plain(TOY_WINDOWED, w, seq)
        scale = np.abs(ref).max()
        pos = 0
        for n in (13, 2, 1, 1, 7, 1, 30, 1, 1, 1, 5, 2, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1):
            got = r.step([StepEntry(0, seq[pos:pos + n], pos, range(n))]).cpu().numpy()
            assert np.abs(got - ref[pos:pos + n]).max() / scale < tol, (dtype, pos, n)
            pos += n
            # the window group holds at most the window plus the current page; the full group everything
            held_w = sum(p >= 0 for p in m.block_table(0, gw))
            held_f = sum(p >= 0 for p in m.block_table(0, gf))
            assert held_w <= (9 + 3) // 4 + 1 and held_f == -(-pos // 4), (pos, held_w, held_f)
            assert m.check() == ""
        assert pos == 87
        r.check_status()
        r.release(0)
        assert m.free_pages(gw) == 24 and m.free_pages(gf) == 24


TOY_SHARED_64 = {"architectures": ["ToyForCausalLM"], "hidden_size": 96, "vocab_size": 211, "inter": 128, "eps": 1e-5,
                 "heads": 4, "kv_heads": 2, "head_dim": 64, "max_pos": 320, "decay": 0.8,
                 # layers 1 and 2 read the keys and values that layer 0 wrote in the same step
                 "mixers": ["attention", "attention", "attention"],
                 "schedule": [[0, None], [1, 0], [2, 0], [1, None]]}


def test_layers_that_read_another_layers_cache_decode_in_bfloat16_through_the_engine():
    """Head size 64, bfloat16, the engine one step ahead, decode steps from captured graphs with
    every kernel launched as a programmatic dependent of the one in front: a layer that keeps
    no cache of its own must still see the key and value that the owning layer wrote for the
    step's own token a few launches earlier.  Logits of every sampled row against the plain
    restatement, for two requests of different lengths beside each other."""
    from kv_cache_optimization_for_llm_b200 import EngineConfig, SamplingParams
    from kv_cache_optimization_for_llm_b200.engine.llm_engine import LLMEngine
    from kv_cache_optimization_for_llm_b200.weights import write_random_model
    from logit_hook import LogitRecorder
    _register_toy()
    d = tempfile.mkdtemp(prefix="kvb200_toy64_")
    write_random_model(d, TOY_SHARED_64, seed=9, std=0.1, storage_dtype="bfloat16")
    w = P.read_safetensors(os.path.join(d, "model.safetensors"))
    eng = LLMEngine(d, EngineConfig(dtype="bfloat16", page_size=16, num_pages=48, max_num_seqs=4,
                                    max_num_batched_tokens=64, max_model_len=320, use_cuda_graphs=True, run_ahead=True))
    rec = LogitRecorder(eng.runner)
    rng = np.random.default_rng(3)
    prompts = [rng.integers(0, 211, n).tolist() for n in (5, 130, 61)]
    ids = [eng.add_request(p, SamplingParams(max_tokens=40, temperature=0.8, seed=i, ignore_eos=True))
           for i, p in enumerate(prompts)]
    while eng.has_unfinished():
        eng.step()
    seqs = {rid: prompts[i] + eng.output(rid) for i, rid in enumerate(ids)}
    n, worst = rec.compare(seqs, lambda rid: _toy_plain(TOY_SHARED_64, w, seqs[rid]), 4e-2, "toy with shared caches")
    assert n >= 3 * 40 and eng.runner._graphs
    assert eng.runner.manager.check() == ""
    print(f"shared caches, head size 64: {n} rows, worst relative error {worst:.3e}")
