"""The Biruvik architecture in the engine against the plain implementation (``plain_biruvik``): each mechanism alone,
whole prompts against token-by-token decoding, portions down to two tokens, mixed batches with pages and state slots
used again, keys far back, at page borders and just inside and just outside a window, memory far back through the
recurrent state, the first tokens of a sequence, long decoding, other sizes (also sizes that are equal or 1), and
greedy generation through ``Engine``.  Configurations and weights are made here; where random numbers would hide a
fault the inputs are planted so that it shows.

CPU tests run the engine with the PyTorch references in place of the kernels (``ref_ops``): they check the plumbing
(configuration, weights, cache, state, batch).  GPU tests run the CUDA kernels."""
import json
import math
import os

import numpy as np
import pytest
import torch

import plain_biruvik as plain
import trace_tools
from tiny_inference_server_b200.api import Engine, SamplingParams
from tiny_inference_server_b200.config import BiruvikConfig, ConfigError, EngineConfig
from tiny_inference_server_b200.registry import build_model, config_from_dict, config_from_folder
from tiny_inference_server_b200.trace import TraceReplayer, make_runner

# ------------------------------------------------------------------------------------------------
# configurations: every size differs between them
# ------------------------------------------------------------------------------------------------


def _diff(heads, kv, dim, vdim, diff=0.25, temp=(0.4, 5), scale=None, window=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "diff": diff, "scale": scale or 2.0 * dim ** -0.5}
    if temp:
        m["q_temp"] = {"coef": temp[0], "every": temp[1]}
    if window:
        m["mask"] = {"size": window}
    return m


def _latent(heads, dim, vdim, rank, window=None, scale=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": rank, "scale": scale or dim ** -0.5}
    if window:
        m["mask"] = {"size": window}
    return m


def _hgrn(heads, dim, vdim):
    return {"heads": heads, "dim": dim, "vdim": vdim}


def _ff(ff, act=None):
    f = {"kind": "dense", "ff": ff}
    if act:
        f["act"] = act
    return f


B1 = dict(architecture="Biruvik", vocab=131, width=64, norm={"eps": 1e-5}, embedding={"scale": 0.7}, logit_softcap=12.0, layers=[
    {"type": "latent_attention", "mixer": _latent(4, 16, 24, 40, window=9), "mlp": _ff(96)},
    {"type": "attention", "mixer": _diff(4, 2, 16, 24), "mlp": None},
    {"type": "hgrn2", "mixer": _hgrn(2, 16, 24), "mlp": _ff(80)},
    {"type": "attention", "mixer": _diff(2, 2, 8, 40, diff=0.6, temp=(1.5, 7), window=13), "mlp": _ff(72, "gelu_tanh")},
    {"type": "latent_attention", "mixer": _latent(2, 24, 8, 16, scale=0.3), "mlp": None},
    {"type": "hgrn2", "mixer": _hgrn(4, 8, 16), "mlp": None},
])
# sizes that are equal or 1 where B1's differ: one head, one kv head, a window of one token, a temperature that grows
# with every position, no temperature, no cap on the logits, an embedding that is not scaled
B2 = dict(architecture="Biruvik", vocab=67, width=32, norm={"eps": 1e-6}, layers=[
    {"type": "hgrn2", "mixer": _hgrn(1, 16, 16), "mlp": _ff(32)},
    {"type": "attention", "mixer": _diff(1, 1, 16, 16, diff=0.5, temp=(0.3, 1)), "mlp": _ff(32)},
    {"type": "latent_attention", "mixer": _latent(1, 16, 16, 16, window=1), "mlp": None},
    {"type": "attention", "mixer": _diff(2, 1, 16, 16, diff=0.1, temp=None), "mlp": None},
    {"type": "latent_attention", "mixer": _latent(1, 16, 16, 16, window=2), "mlp": _ff(32, "silu")},
])
# sizes that fit no vector, tile or alignment: every kernel's plain path
B3 = dict(architecture="Biruvik", vocab=53, width=40, norm={"eps": 1e-6}, embedding={"scale": 1.3}, logit_softcap=5.0, layers=[
    {"type": "attention", "mixer": _diff(3, 1, 10, 6, temp=(0.2, 3)), "mlp": _ff(27)},
    {"type": "latent_attention", "mixer": _latent(3, 10, 7, 22, window=7), "mlp": _ff(13)},
    {"type": "hgrn2", "mixer": _hgrn(3, 10, 6), "mlp": None},
    {"type": "attention", "mixer": _diff(3, 3, 6, 10, diff=0.4), "mlp": None},
])
# sizes of the fast paths: attention on the tensor cores (a window that ends at a tile of keys and one that does not),
# the recurrence with a head's columns split over CTAs
B4 = dict(architecture="Biruvik", vocab=90, width=96, norm={"eps": 1e-5}, embedding={"scale": 0.5}, logit_softcap=30.0, layers=[
    {"type": "attention", "mixer": _diff(4, 1, 32, 32, temp=(0.3, 16)), "mlp": _ff(128)},
    {"type": "latent_attention", "mixer": _latent(8, 32, 16, 48, window=64), "mlp": None},
    {"type": "hgrn2", "mixer": _hgrn(2, 64, 64), "mlp": _ff(128)},
    {"type": "latent_attention", "mixer": _latent(2, 16, 32, 96, window=37), "mlp": _ff(64)},
    {"type": "attention", "mixer": _diff(6, 2, 16, 64, diff=0.2, temp=(0.5, 32)), "mlp": None},
    {"type": "hgrn2", "mixer": _hgrn(1, 128, 32), "mlp": None},
])
CONFIGS = {"B1": (B1, 16), "B2": (B2, 8), "B3": (B3, 12), "B4": (B4, 16)}
LENGTHS = {"B1": [1, 2, 3, 30, 75, 41, 9, 60], "B2": [1, 5, 40, 33, 17, 64], "B3": [2, 4, 50, 90, 23, 37],
           "B4": [3, 1, 45, 20, 150]}


def make_tensors(cfg, seed):
    """Weights of a size that makes every mechanism matter: projections of unit gain (queries, keys and the
    compressed projection sharper), norms behind the sublayers that let an update through at about half the size of
    the stream, gates' lower bounds all over (0, 0.9); rounded to bfloat16 so that both precisions and the plain
    implementation hold the same numbers."""
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, spec in build_model(cfg).expected_tensors().items():
        shape = tuple(spec.shape)
        leaf = name.split(".", 1)[1] if name.startswith("l") else name
        rnd = torch.randn(shape, generator=gen)
        uni = torch.rand(shape, generator=gen)
        if name == "embed":
            t = rnd
        elif leaf in ("norm1b", "norm2b"):
            t = 0.5 + rnd * 0.1
        elif leaf in ("norm1", "norm2", "mix.norm", "mix.dkv.norm", "mix.q.norm", "mix.k.norm") or name == "final.norm":
            t = 1.0 + rnd * 0.2
        elif leaf in ("mix.lq1", "mix.lk1", "mix.lq2", "mix.lk2"):
            t = rnd * 0.4
        elif leaf == "mix.lower":
            t = uni * 0.9
        elif leaf.endswith(".b"):
            t = rnd * 0.5
        elif len(shape) == 2:
            gain = 2.0 if leaf in ("mix.q", "mix.k", "mix.dkv", "mix.f", "mix.g") else 1.0
            t = rnd * gain / math.sqrt(shape[1])
        else:
            raise AssertionError(f"no rule for {name} {shape}")
        out[name] = t.to(torch.bfloat16).contiguous()
    return out


def make_folder(raw, seed, folder):
    from safetensors.torch import save_file
    cfg = config_from_dict(json.loads(json.dumps(raw)))
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg.to_dict(), f)
    save_file(make_tensors(cfg, seed), os.path.join(folder, "model.safetensors"))
    return folder


_cache = {}


def _setup(name, tmp_path_factory):
    if name not in _cache:
        raw, page = CONFIGS[name]
        folder = make_folder(raw, 23 + ord(name[-1]), str(tmp_path_factory.mktemp(f"biruvik{name}")))
        c, W = plain.read_config(folder), plain.read_weights(folder)
        g = torch.Generator().manual_seed(5)
        seqs = {f"r{i}": torch.randint(0, raw["vocab"], (n,), generator=g).tolist() for i, n in enumerate(LENGTHS[name])}
        ref = {rid: plain.plain_forward(c, W, toks).numpy() for rid, toks in seqs.items()}
        _cache[name] = (raw, page, folder, seqs, ref, c, W)
    return _cache[name]


def rel_err(got, ref):
    """Difference of two rows of logits, mean taken off, root mean square, over that of the reference."""
    d = np.asarray(got, dtype=np.float64) - ref
    d = d - d.mean()
    r = ref - ref.mean()
    return float(np.sqrt((d * d).mean()) / max(np.sqrt((r * r).mean()), 1e-9))


TOL = {"float32": 2e-4, "bfloat16": 6e-2}
#: In float32 every position agrees.  In bfloat16 one position in a hundred may differ by more than the tolerance (by less
#: than 1): among hundreds of positions of random weights a few are ill-conditioned (the difference of two maps that
#: nearly cancel, then divided by its own size), and there rounding the activations between kernels moves the logits
#: as far as the kernels do.
BF16_OUTLIERS = {"float32": 0.0, "bfloat16": 0.01}


def _steps(mode, seqs, max_live=4):
    if mode == "whole":
        return trace_tools.trace_whole(seqs)
    if mode == "tail":
        return trace_tools.trace_tail(seqs, tail=32)
    if mode == "chunks":
        return trace_tools.trace_chunks(seqs)
    return trace_tools.trace_mixed(seqs, max_live=max_live)


def _replay_and_compare(raw, page, folder, seqs, ref, steps, out_dir, dtype, device, tol, max_live=4, poison=False,
                        shuffle=False, outliers=0.0):
    """``outliers``: the share of positions that may exceed the tolerance (none of them by more than 1)."""
    runner = make_runner(folder, dtype, trace_tools.max_live_tokens(steps, round_to=64), page_size=page, device=device,
                         max_live=max_live, debug_poison=poison)
    if shuffle:
        import random
        for g in runner.cache.groups:
            g.pool.shuffle(random.Random(3))
    TraceReplayer(runner, out_dir).run(json.dumps(s) for s in steps)
    runner.cache.check()
    assert runner.cache.drained(), "pages or slots were not given back"
    got = trace_tools.gather(steps, out_dir, raw["vocab"])
    worst, over, total = 0.0, [], sum(len(t) for t in seqs.values())
    for rid, toks in seqs.items():
        for p in range(len(toks)):
            e = rel_err(got[rid][p], ref[rid][p])
            if e >= tol:
                over.append((rid, p, e))
                assert e < 1.0 and len(over) <= outliers * total, \
                    f"logits of {rid} at position {p}: relative error {e} (first wrong place; over the tolerance so far: {over})"
            worst = max(worst, e)
    return runner, worst


# ------------------------------------------------------------------------------------------------
# configuration and weights (CPU)
# ------------------------------------------------------------------------------------------------

def test_config_round_trip_and_tensor_names(tmp_path):
    folder = make_folder(B1, 1, str(tmp_path / "m"))
    cfg = config_from_folder(folder)
    assert isinstance(cfg, BiruvikConfig)
    again = config_from_dict(cfg.to_dict())
    assert again.to_dict() == cfg.to_dict()
    specs = build_model(cfg).expected_tensors()
    names = set(specs)
    assert {"embed", "final.norm", "head", "l0.norm1", "l0.norm1b", "l0.norm2", "l0.norm2b", "l0.mix.dkv.norm", "l0.mix.g",
            "l0.mix.uk", "l1.mix.q.b", "l1.mix.lq2", "l1.mix.k.norm", "l2.mix.lower", "l2.mix.f.b", "l2.mix.norm",
            "l2.mlp.up", "l2.mlp.down"} <= names
    assert "l1.norm2" not in names and "l1.norm2b" not in names and "l1.mlp.up" not in names and "l0.mix.sink" not in names
    shapes = {n: tuple(s.shape) for n, s in specs.items()}
    assert shapes["l0.norm1"] == () and shapes["final.norm"] == ()
    assert shapes["l1.mix.q"] == (4 * 2 * 16, 64) and shapes["l1.mix.k"] == (2 * 2 * 16, 64) and shapes["l1.mix.v"] == (2 * 24, 64)
    assert shapes["l1.mix.o"] == (64, 4 * 24) and shapes["l1.mix.q.norm"] == (16,) and shapes["l1.mix.lk1"] == (16,)
    assert shapes["l0.mix.dkv"] == (40, 64) and shapes["l0.mix.uv"] == (4 * 24, 40) and shapes["l0.mix.g"] == (4, 64)
    assert shapes["l2.mix.f"] == (32, 64) and shapes["l2.mix.v"] == (48, 64) and shapes["l2.mix.norm"] == (24,)


def test_config_errors_name_the_problem():
    def broken(change):
        bad = json.loads(json.dumps(B1))
        change(bad)
        return bad

    with pytest.raises(ConfigError, match="layers\\[0\\].type"):
        config_from_dict(broken(lambda c: c["layers"][0].update(type="conv_only")))
    with pytest.raises(ConfigError, match="not a multiple"):
        config_from_dict(broken(lambda c: c["layers"][1]["mixer"].update(heads=3)))
    with pytest.raises(ConfigError, match="diff is missing"):
        config_from_dict(broken(lambda c: c["layers"][1]["mixer"].pop("diff")))
    with pytest.raises(ConfigError, match="q_temp"):
        config_from_dict(broken(lambda c: c["layers"][1]["mixer"].update(q_temp={"coef": 0.1, "every": 0})))
    with pytest.raises(ConfigError, match="kv_rank"):
        config_from_dict(broken(lambda c: c["layers"][0]["mixer"].pop("kv_rank")))
    with pytest.raises(ConfigError, match="mask.size"):
        config_from_dict(broken(lambda c: c["layers"][0]["mixer"].update(mask={"size": 0})))
    with pytest.raises(ConfigError, match="mlp.kind"):
        config_from_dict(broken(lambda c: c["layers"][0]["mlp"].update(kind="moe")))
    with pytest.raises(ConfigError, match="missing keys: width"):
        config_from_dict(broken(lambda c: c.pop("width")))


def test_a_missing_or_misshapen_tensor_is_named(tmp_path):
    from safetensors.torch import load_file, save_file
    folder = make_folder(B2, 2, str(tmp_path / "m"))
    path = os.path.join(folder, "model.safetensors")
    good = load_file(path)
    eng = EngineConfig(dtype="float32", page_size=8, num_pages=4, max_batch=1, device="cpu", cuda_graphs=False)
    bad = dict(good)
    bad.pop("l0.mix.lower")
    save_file(bad, path)
    with pytest.raises(Exception, match="l0.mix.lower"):
        Engine.from_folder(folder, eng)
    bad = dict(good)
    bad["l1.norm1b"] = torch.ones(32, dtype=torch.bfloat16)         # a norm's weight is one number
    save_file(bad, path)
    with pytest.raises(Exception, match="l1.norm1b"):
        Engine.from_folder(folder, eng)


# ------------------------------------------------------------------------------------------------
# the plain implementation against itself: the same mechanism written a second way
# ------------------------------------------------------------------------------------------------

def _some_weights(cfg_raw, seed):
    cfg = config_from_dict(json.loads(json.dumps(cfg_raw)))
    return {k: v.double() for k, v in make_tensors(cfg, seed).items()}


def test_plain_mixers_position_by_position():
    """Every mixer of the plain implementation, which works on whole sequences with masks, equals a loop that takes one
    position at a time and adds up the keys it may see one by one."""
    W = _some_weights(B1, 3)
    eps = B1["norm"]["eps"]
    torch.manual_seed(0)
    L = 31
    u = torch.randn(L, B1["width"], dtype=torch.float64)
    # latent attention with a window of 9
    m, p = B1["layers"][0]["mixer"], "l0.mix."
    H, dim, vdim, win = m["heads"], m["dim"], m["vdim"], m["mask"]["size"]
    c = plain.rms(u @ W[p + "dkv"].T, eps) * W[p + "dkv.norm"]
    heads = torch.zeros(L, H, vdim, dtype=torch.float64)
    for i in range(L):
        for h in range(H):
            q = (W[p + "q"] @ u[i])[h * dim:(h + 1) * dim]
            num, den = torch.zeros(vdim, dtype=torch.float64), 0.0
            for j in range(max(0, i - win + 1), i + 1):
                e = math.exp(float(q @ (W[p + "uk"] @ c[j])[h * dim:(h + 1) * dim]) * m["scale"])
                num, den = num + e * (W[p + "uv"] @ c[j])[h * vdim:(h + 1) * vdim], den + e
            heads[i, h] = num / den * torch.sigmoid(W[p + "g"][h] @ u[i])
    assert float((plain.latent_window_attention(u, W, p, m, eps) - heads.reshape(L, -1) @ W[p + "o"].T).abs().max()) < 1e-9
    # differential attention, two kv heads
    m, p = B1["layers"][1]["mixer"], "l1.mix."
    H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    lam = math.exp(float(W[p + "lq1"] @ W[p + "lk1"])) - math.exp(float(W[p + "lq2"] @ W[p + "lk2"])) + m["diff"]
    qs, ks, vs = u @ W[p + "q"].T + W[p + "q.b"], u @ W[p + "k"].T + W[p + "k.b"], u @ W[p + "v"].T + W[p + "v.b"]
    heads = torch.zeros(L, H, vdim, dtype=torch.float64)
    for i in range(L):
        temp = 1.0 + m["q_temp"]["coef"] * math.log((i + 1) // m["q_temp"]["every"] + 1)
        for h in range(H):
            g = h // (H // G)
            maps = []
            for mp in range(2):
                q = qs[i, (2 * h + mp) * dim:(2 * h + mp + 1) * dim]
                q = q / math.sqrt(float((q * q).mean()) + eps) * W[p + "q.norm"] * temp
                num, den = torch.zeros(vdim, dtype=torch.float64), 0.0
                for j in range(i + 1):
                    k = ks[j, (2 * g + mp) * dim:(2 * g + mp + 1) * dim]
                    k = k / math.sqrt(float((k * k).mean()) + eps) * W[p + "k.norm"]
                    e = math.exp(float(q @ k) * m["scale"])
                    num, den = num + e * vs[j, g * vdim:(g + 1) * vdim], den + e
                maps.append(num / den)
            o = maps[0] - lam * maps[1]
            heads[i, h] = o / math.sqrt(float((o * o).mean()) + eps) * (1.0 - m["diff"])
    assert float((plain.differential_attention(u, W, p, m, eps) - heads.reshape(L, -1) @ W[p + "o"].T).abs().max()) < 1e-9


def test_plain_recurrence_carries_its_state():
    """The recurrence over a sequence equals the recurrence over its first part, then over the rest from the state the
    first part left; and, written out for one channel, a state entry is the gate-weighted sum of the values."""
    W = _some_weights(B1, 4)
    eps = B1["norm"]["eps"]
    m, p = B1["layers"][2]["mixer"], "l2.mix."
    H, dim, vdim = m["heads"], m["dim"], m["vdim"]
    torch.manual_seed(1)
    L = 40
    u = torch.randn(L, B1["width"], dtype=torch.float64)
    whole = plain.gated_forget_recurrence(u, W, p, m, eps)
    low = W[p + "lower"]
    f = low + (1 - low) * torch.sigmoid(u @ W[p + "f"].T + W[p + "f.b"])
    v = u @ W[p + "v"].T
    assert bool((f >= low).all()) and bool((f <= 1).all())
    S = torch.zeros(H, dim, vdim, dtype=torch.float64)
    for t in range(17):
        S = f[t].view(H, dim, 1) * S + (1 - f[t]).view(H, dim, 1) * v[t].view(H, 1, vdim)
    rest = plain.gated_forget_recurrence(u[17:], W, p, m, eps, state=S)
    assert float((whole[17:] - rest).abs().max()) < 1e-10
    # one entry of the state after 17 tokens: sum_s (1 - f_s) v_s prod_{r > s} f_r
    h, d, e = 1, 3, 5
    ch = h * dim + d
    want = sum(float((1 - f[s, ch]) * v[s, h * vdim + e] * torch.prod(f[s + 1:17, ch])) for s in range(17))
    assert abs(float(S[h, d, e]) - want) < 1e-12


# ------------------------------------------------------------------------------------------------
# the engine's plumbing on the CPU
# ------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("name", ["B1", "B2", "B3", "B4"])
@pytest.mark.parametrize("mode", ["whole", "tail", "chunks", "mixed"])
def test_replay_cpu(name, mode, tmp_path, tmp_path_factory, ref_ops):
    raw, page, folder, seqs, ref, _, _ = _setup(name, tmp_path_factory)
    steps = _steps(mode, seqs, max_live=3)
    _replay_and_compare(raw, page, folder, seqs, ref, steps, str(tmp_path / "out"), "float32", "cpu", 1e-4, max_live=3,
                        poison=(mode == "mixed"))


def test_layers_of_the_stream_cpu(tmp_path_factory, ref_ops):
    """The residual stream after every layer, read from the model's blocks one by one, against the plain layers."""
    raw, page, folder, seqs, _, c, W = _setup("B1", tmp_path_factory)
    toks = seqs["r5"]
    _, layers = plain.plain_forward(c, W, toks, return_layers=True)
    runner = make_runner(folder, "float32", 64, page_size=page, device="cpu", max_live=1)
    from tiny_inference_server_b200.engine.batch import StepEntry
    from tiny_inference_server_b200.parts.stream import ResidualStream
    seen = []
    for e in runner.model.entries:
        inner = e.block.forward

        def spy(stream, step, binding, *a, _inner=inner, **kw):
            _inner(stream, step, binding, *a, **kw)
            seen.append(stream.flush().clone())
        e.block.forward = spy
    slot = runner.add_request()
    runner.step([StepEntry(slot, list(toks), [len(toks) - 1])])
    runner.release(slot)
    assert len(seen) == len(c["layers"])
    for i, (got, want) in enumerate(zip(seen, layers)):
        err = float((got.double() - want).abs().max() / want.abs().max())
        assert err < 1e-4, f"stream after layer {i} ({c['layers'][i]['type']}): {err}"


def plain_greedy(c, W, prompt, new):
    ids = list(prompt)
    for _ in range(new):
        ids.append(int(plain.plain_forward(c, W, ids)[-1].argmax()))
    return ids[len(prompt):]


def test_generate_cpu(tmp_path, tmp_path_factory, ref_ops):
    raw, page, folder, seqs, ref, c, W = _setup("B2", tmp_path_factory)
    prompts = [seqs["r1"], seqs["r4"], seqs["r0"]]
    want = [plain_greedy(c, W, p, 6) for p in prompts]
    sp = SamplingParams(max_new_tokens=6, temperature=0.0, ignore_eos=True)
    eng = Engine.from_folder(folder, EngineConfig(dtype="float32", page_size=page, num_pages=32, max_batch=2,
                                                  max_tokens_per_step=7, device="cpu", cuda_graphs=False))
    assert eng.generate(prompts, sp) == want
    assert eng.runner.cache.drained()
