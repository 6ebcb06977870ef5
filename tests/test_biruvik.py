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
B4 = dict(architecture="Biruvik", vocab=90, width=96, norm={"eps": 2e-6}, embedding={"scale": 0.8}, logit_softcap=20.0, layers=[
    {"type": "attention", "mixer": _diff(4, 1, 32, 32, temp=(0.35, 16)), "mlp": _ff(128)},
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
#: In float32 every position agrees.  In bfloat16 two positions in a hundred may differ by more than the tolerance (by less
#: than 1): among hundreds of positions of random weights a few are ill-conditioned (the difference of two maps that
#: nearly cancel, then divided by its own size; a softmax sharpened fourfold by the query temperature), and there
#: rounding the activations between kernels moves the logits as far as the kernels do: the PyTorch references in place
#: of the kernels, run in bfloat16, differ from the plain implementation at the same positions by the same amounts.
BF16_OUTLIERS = {"float32": 0.0, "bfloat16": 0.02}


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


# ------------------------------------------------------------------------------------------------
# GPU: each mechanism alone against the plain functions
# ------------------------------------------------------------------------------------------------

gpu = pytest.mark.gpu
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def _close(got, ref, tol, what):
    got = got.detach().double().cpu()
    err = float((got - ref).abs().max() / max(float(ref.abs().max()), 1e-9))
    assert err < tol, f"{what}: relative error {err}"


def _rows(cuts, slots):
    """row_slot and row_last of a step that holds ``cuts[i]`` rows of slot ``slots[i]``."""
    row_slot, row_last = [], []
    for n, s in zip(cuts, slots):
        first = len(row_slot)
        row_slot += [s] * n
        row_last += [first + n - 1] * n
    i32 = dict(dtype=torch.int32, device="cuda")
    return torch.tensor(row_slot, **i32), torch.tensor(row_last, **i32)


class _Step:
    """What an attention kernel asks of a step, for one request's portion outside the engine."""

    def __init__(self, positions, row_slot, decode_only=False):
        self.positions, self.row_slot, self.decode_only = positions, row_slot, decode_only
        self.max_position = int(positions.max())

    def plan(self, planner):
        return planner.infer(self.positions, self.row_slot)


def _selectors(width, parts):
    """Projections that pick columns: ``parts`` = [(name, columns)], side by side from column 0.  With them a plain
    mixer reads its queries, keys and values straight out of its input, so that a test can plant them."""
    W, at = {}, 0
    for name, n in parts:
        W[name] = torch.zeros(n, width, dtype=torch.float64)
        W[name][torch.arange(n), at + torch.arange(n)] = 1.0
        at += n
    return W


def _scattered_pages(L, page, slots=3, slot=1, extra=3):
    n_pages = (L + page - 1) // page + extra
    perm = torch.randperm(n_pages)[: (L + page - 1) // page].to(torch.int32)
    table = torch.full((slots, len(perm) + 2), -1, dtype=torch.int32)
    table[slot, :len(perm)] = perm
    return n_pages, perm, table.cuda()


def _portions(L, cuts, alone=4):
    """(first row, rows) of portions that follow ``cuts`` in turn; the last ``alone`` rows come one by one."""
    fed, i = 0, 0
    while fed < L:
        n = min(cuts[i % len(cuts)], max(1, L - alone - fed)) if fed < L - alone else 1
        yield i, fed, n
        i += 1
        fed += n


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,kd,vd", [(2, 16, 24), (1, 16, 16), (3, 10, 6), (2, 64, 64), (1, 128, 32), (4, 32, 96), (2, 32, 128),
                                      (1, 256, 256), (2, 160, 224), (2, 16, 320), (1, 40, 520)])
def test_forget_gate_recurrence_in_portions_and_far_memory(dtype, H, kd, vd):
    """Two sequences side by side in slots 2 and 0, in portions of 1..70 rows, equal the plain recurrence over the
    whole sequences.  Head 0's gate is shut (f = 1: nothing forgotten, nothing written) but for position 1, where it
    is wide open: what that token wrote is what the head reads 250 tokens later.  The last head's gate stays near
    its lower bound of zero and forgets within a few tokens."""
    from tiny_inference_server_b200.kernels import ops
    torch.manual_seed(kd * 3 + vd)
    L = 260
    nq, nv = H * kd, H * vd
    eps = 1e-5
    m = {"heads": H, "dim": kd, "vdim": vd}
    W = _selectors(2 * nq + nv, [("q", nq), ("v", nv), ("f", nq)])
    W["o"] = torch.eye(nv, dtype=torch.float64)
    lower = torch.rand(nq) * 0.9
    lower[:kd] = 0.0
    if H > 1:
        lower[-kd:] = 0.0
    f_bias = torch.randn(nq) * 0.5
    f_bias[:kd] = 0.0
    norm_w = 1 + 0.2 * torch.randn(vd)
    W.update({"lower": lower.double(), "f.b": f_bias.double(), "norm": norm_w.double()})
    seqs, refs, finals = [], [], []
    for s in range(2):
        u = torch.randn(L, 2 * nq + nv)
        u[:, nq + nv:nq + nv + kd] = 20.0                  # head 0: shut ...
        u[1, nq + nv:nq + nv + kd] = -20.0                 # ... but for position 1
        u[L - 3, :kd] = u[L - 3, :kd].abs() + 0.5          # a query that reads it with a clear sign
        if H > 1:
            u[:, -kd:] = -3.0
        u = u.to(DT[dtype])
        seqs.append(u)
        ref = plain.gated_forget_recurrence(u.double(), W, "", m, eps)
        far = plain.rms(u[1, nq:nq + vd].double(), eps) * norm_w.double()
        assert float((ref[L - 3, :vd] - far).abs().max()) < 1e-3 * float(far.abs().max()), "the planted memory does not show"
        refs.append(ref)
        f = (W["lower"] + (1 - W["lower"]) * torch.sigmoid(u.double()[:, nq + nv:] + W["f.b"])).view(L, H, kd)
        v = u.double()[:, nq:nq + nv].view(L, H, vd)
        S = torch.zeros(H, kd, vd, dtype=torch.float64)
        for t in range(L):
            S = f[t][:, :, None] * S + (1 - f[t])[:, :, None] * v[t][:, None, :]
        finals.append(S.reshape(-1))
    state = torch.zeros(3, nq * vd + 5, device="cuda")
    got = [torch.zeros(L, nv, dtype=DT[dtype], device="cuda") for _ in range(2)]
    fed = [0, 0]
    sizes = [(1, 2), (2, 1), (17, 3), (1, 1), (33, 70), (70, 2), (2, 16), (16, 5), (5, 64), (64, 33)]
    i = 0
    while min(fed) < L:
        a, b = sizes[i % len(sizes)]
        i += 1
        cuts = [min(a, L - fed[0]), min(b, L - fed[1])]
        parts = [(s, c) for s, c in zip((0, 1), cuts) if c > 0]
        rows = torch.cat([seqs[s][fed[s]:fed[s] + c] for s, c in parts]).cuda()
        row_slot, row_last = _rows([c for _, c in parts], [(2, 0)[s] for s, _ in parts])
        out = torch.empty(rows.shape[0], nv, dtype=DT[dtype], device="cuda")
        ops.forget_gate_recurrence(rows[:, :nq + nv], rows[:, nq + nv:], lower.cuda(), f_bias.cuda(), norm_w.cuda(), eps, state,
                                   out, row_slot, row_last, H, kd, vd, requests=len(parts) if i % 2 else None)
        at = 0
        for s, c in parts:
            got[s][fed[s]:fed[s] + c] = out[at:at + c]
            at += c
            fed[s] += c
    for s in range(2):
        _close(got[s], refs[s], 3e-2 if dtype == "bfloat16" else 1e-4, "forget-gate recurrence")
        _close(state[(2, 0)[s], :nq * vd], finals[s], 2e-2 if dtype == "bfloat16" else 1e-4, "state")
    assert float(state[1].abs().max()) == 0 and float(state[:, nq * vd:].abs().max()) == 0


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,dim,vd,page,window,temp", [(4, 2, 16, 24, 16, None, (0.4, 5)), (2, 2, 8, 40, 4, 13, (1.5, 7)),
                                                         (3, 1, 10, 6, 12, None, (0.2, 3)), (4, 1, 32, 48, 16, None, (0.35, 48)),
                                                         (1, 1, 16, 16, 8, None, None), (6, 2, 16, 64, 16, 70, (0.5, 1)),
                                                         (2, 1, 64, 32, 32, None, (0.25, 100))])
def test_differential_attention_and_a_key_far_back(dtype, H, G, dim, vd, page, window, temp):
    """Bias, norm per head and map, query temperature and the cache rows; two maps over the same values; their
    combination.  In portions and single rows over scattered pages.  Map 1 of head 0 of some rows near the end asks
    for the key of position 3, several hundred keys back (or, with a window, for the keys just inside and just outside
    it), and for the keys at the last and first place of a page; map 2 of those rows does not, so a kernel that mixed
    the maps up, or lost the far key, gives another row."""
    from tiny_inference_server_b200.kernels import ops
    torch.manual_seed(H * 10 + dim)
    L = 333
    nq, nk, nv = H * 2 * dim, G * 2 * dim, G * vd
    eps, scale, diff = 1e-5, 5.0 * dim ** -0.5, 0.3
    m = {"heads": H, "kv_heads": G, "dim": dim, "vdim": vd, "diff": diff, "scale": scale}
    if temp:
        m["q_temp"] = {"coef": temp[0], "every": temp[1]}
    if window:
        m["mask"] = {"size": window}
    W = _selectors(nq + nk + nv, [("q", nq), ("k", nk), ("v", nv)])
    W["o"] = torch.eye(H * vd, dtype=torch.float64)
    bias = torch.randn(nq + nk + nv) * 0.3
    W.update({"q.b": bias[:nq].double(), "k.b": bias[nq:nq + nk].double(), "v.b": bias[nq + nk:].double()})
    qw, kw = 1 + 0.2 * torch.randn(dim), 1 + 0.2 * torch.randn(dim)
    W.update({"q.norm": qw.double(), "k.norm": kw.double()})
    for name in ("lq1", "lk1", "lq2", "lk2"):
        W[name] = (torch.randn(dim) * 0.4).double()
    lam = plain.differential_lambda(W, "", diff)
    u = torch.randn(L, nq + nk + nv)
    if window:
        asked = {L - 1: L - window, L - 2: L - 2 - window, L - 40: L - 39 - window, L - 41: L - 41 - window}
    else:
        asked = {L - 1: 2, L - 2: page - 1, L - 5: 2 * page, L - 40: 5}
    # map 1 of kv head 0: key channel i is empty in every key but the i-th asked one, which is nothing else; the asking
    # row's query (map 1 of head 0) is that channel alone.  (What the bias adds is taken off first.)
    u[:, nq:nq + len(asked)] = -bias[nq:nq + len(asked)]
    for i, (r_, j) in enumerate(asked.items()):
        u[j, nq:nq + dim] = -bias[nq:nq + dim]
        u[j, nq + i] += 4.0
        u[r_, :dim] = -bias[:dim]
        u[r_, i] += 4.0 * float(torch.sign(qw[i] * kw[i]))
    u = u.to(DT[dtype])
    ref = plain.differential_attention(u.double(), W, "", m, eps)
    # the asked key carries map 1 of head 0 where the row may see it, and no weight where it may not
    q = plain.rms((u.double()[:, :nq] + W["q.b"]).view(L, H, 2, dim), eps) * W["q.norm"]
    k = plain.rms((u.double()[:, nq:nq + nk] + W["k.b"]).view(L, G, 2, dim), eps) * W["k.norm"]
    for r_, j in asked.items():
        t = float(plain.query_temperature(torch.tensor([r_]), temp[0], temp[1])) if temp else 1.0
        lo = max(0, r_ - window + 1) if window else 0
        s = (k[lo:r_ + 1, 0, 0] @ q[r_, 0, 0]) * scale * t
        w = torch.softmax(s, 0)
        if j >= lo:
            assert float(w[j - lo]) > 0.5, (r_, j, float(w[j - lo]))
        else:
            assert float((k[j, 0, 0] @ q[r_, 0, 0]) * scale * t) > float(s.max()) + 3.0, "the key outside would have won"
    n_pages, perm, table = _scattered_pages(L, page)
    kp = torch.full((n_pages, G, page, 2 * dim), 1e4, dtype=DT[dtype], device="cuda")
    vp = torch.full((n_pages, G, page, vd), 1e4, dtype=DT[dtype], device="cuda")
    fault = torch.zeros(4, dtype=torch.int32, device="cuda")
    got = torch.zeros(L, H * vd, dtype=DT[dtype], device="cuda")
    cuda_w = lambda t: t.float().cuda().contiguous()
    for i, fed, n in _portions(L, [5, 2, 1, 1, 30, 2, 64, 100]):
        rows = slice(fed, fed + n)
        pos = torch.arange(fed, fed + n, dtype=torch.int32, device="cuda")
        slot = torch.full((n,), 1, dtype=torch.int32, device="cuda")
        qbuf = torch.full((n, H * 2 * 2 * dim), 7.0, dtype=DT[dtype], device="cuda")
        ops.head_norm_store(u[rows].cuda(), H, G, 2, dim, vd, cuda_w(bias), cuda_w(qw), cuda_w(kw), eps,
                            temp[0] if temp else 0.0, temp[1] if temp else 0, qbuf, kp, vp, table, pos, slot, page, fault)
        maps = torch.empty(n, H * 2 * vd, dtype=DT[dtype], device="cuda")
        ops.window_attention(qbuf, None, maps, kp, vp, table, pos, slot, H * 2, page, window, scale, None, None, fault,
                             step=_Step(pos, slot, decode_only=(n == 1 and i % 2 == 0)) if n != 2 else None)
        out = torch.empty(n, H * vd, dtype=DT[dtype], device="cuda")
        ops.diff_combine(maps, lam, eps, 1.0 - diff, out, H, vd, slot)
        got[rows] = out
    assert int(fault[0]) == 0
    stored = torch.stack([kp[int(perm[p // page]), :, p % page] for p in range(L)])
    _close(stored, k.reshape(L, G, 2 * dim), 2e-2 if dtype == "bfloat16" else 1e-5, "key rows of the cache")
    # bfloat16 rounds the two maps before they are subtracted and the difference is divided by its own size: rows whose maps
    # nearly cancel are ill-conditioned, so the share of rows beyond the tolerance is bounded, not the worst row
    err = (got.double().cpu() - ref).abs().amax(-1) / float(ref.abs().max())
    if dtype == "float32":
        assert float(err.max()) < 1e-4, f"differential attention: {float(err.max())} at row {int(err.argmax())}"
    else:
        assert float((err > 5e-2).double().mean()) < 0.04 and float(err.max()) < 0.2, \
            f"differential attention: {float(err.max())} at row {int(err.argmax())}, {int((err > 5e-2).sum())} rows over"


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,dim,vd,rank,page,window", [(4, 16, 24, 40, 16, 9), (2, 24, 8, 16, 4, None), (3, 10, 7, 22, 12, 7),
                                                       (8, 32, 16, 48, 16, 64), (1, 16, 16, 16, 8, 1), (2, 16, 32, 96, 16, 37),
                                                       (4, 32, 32, 64, 16, 200), (2, 8, 16, 32, 8, 2)])
def test_windowed_latent_attention_with_head_gates(dtype, H, dim, vd, rank, page, window):
    """The compressed vector's norm and its cache rows without a rotated slice, the queries taken through the key
    expansion, attention over a window of the compressed rows with one sigmoid gate per head, the value expansion; in
    portions and single rows over scattered pages.  Head 0 of some rows near the end asks for the key at the window's
    far edge, and of others for the key one place beyond it (without a window: for keys several hundred places back
    and at the edges of a page)."""
    from tiny_inference_server_b200.kernels import ops
    torch.manual_seed(H * 10 + rank)
    L = 333
    nq = H * dim
    eps, scale = 1e-5, dim ** -0.5
    m = {"heads": H, "dim": dim, "vdim": vd, "kv_rank": rank, "scale": scale}
    if window:
        m["mask"] = {"size": window}
        asked = {L - 1: L - window, L - 2: L - 2 - window, L - 40: L - 39 - window, L - 41: L - 41 - window}
    else:
        asked = {L - 1: 2, L - 2: page - 1, L - 5: 2 * page, L - 40: 5}
    W = _selectors(nq + rank + H, [("q", nq), ("dkv", rank), ("g", H)])
    W["o"] = torch.eye(H * vd, dtype=torch.float64)
    cw = 1 + 0.2 * torch.randn(rank)
    uk = torch.randn(H * dim, rank) / math.sqrt(rank)
    uv = torch.randn(H * vd, rank) / math.sqrt(rank)
    # head 0's key channel i is the compressed vector's channel i and nothing else (i below the number of asked keys)
    na = len(asked)
    uk[:na, :] = 0.0
    uk[:dim, :na] = 0.0
    uk[torch.arange(na), torch.arange(na)] = 1.0
    uk, uv = uk.to(torch.bfloat16).float(), uv.to(torch.bfloat16).float()
    W.update({"dkv.norm": cw.double(), "uk": uk.double(), "uv": uv.double()})
    u = torch.randn(L, nq + rank + H)
    u[:, nq + rank:] *= 2.0
    u[:, nq:nq + na] = 0.0                                  # that channel is empty in every compressed vector ...
    for i, (r_, j) in enumerate(asked.items()):
        u[j, nq:nq + rank] = 0.0
        u[j, nq + i] = 1.0                                  # ... but the asked one, which is nothing else
        u[r_, :dim] = 0.0
        u[r_, i] = 12.0 / (scale * math.sqrt(rank) * float(cw[i]))
    u = u.to(DT[dtype])
    ref = plain.latent_window_attention(u.double(), W, "", m, eps)
    c = plain.rms(u.double()[:, nq:nq + rank], eps) * W["dkv.norm"]
    k0 = c @ W["uk"][:dim].T
    for r_, j in asked.items():
        lo = max(0, r_ - window + 1) if window else 0
        s = (k0[lo:r_ + 1] @ u.double()[r_, :dim]) * scale
        if j >= lo:
            assert float(torch.softmax(s, 0)[j - lo]) > 0.5, (r_, j)
        else:
            assert float(k0[j] @ u.double()[r_, :dim]) * scale > float(s.max()) + 3.0, "the key outside would have won"
    n_pages, perm, table = _scattered_pages(L, page)
    kp = torch.full((n_pages, 1, page, rank), 1e4, dtype=DT[dtype], device="cuda")
    fault = torch.zeros(4, dtype=torch.int32, device="cuda")
    w_uk = uk.to(DT[dtype]).reshape(H, dim, rank).cuda().contiguous()
    w_uv = uv.to(DT[dtype]).reshape(H, vd, rank).transpose(1, 2).cuda().contiguous()
    got = torch.zeros(L, H * vd, dtype=DT[dtype], device="cuda")
    for i, fed, n in _portions(L, [5, 2, 1, 1, 30, 2, 64, 100]):
        rows = slice(fed, fed + n)
        pos = torch.arange(fed, fed + n, dtype=torch.int32, device="cuda")
        slot = torch.full((n,), 1, dtype=torch.int32, device="cuda")
        proj = u[rows].cuda()
        q = torch.empty(n, H * rank, dtype=DT[dtype], device="cuda")
        ops.latent_prepare(proj, nq, H, dim, 0, rank, cw.cuda(), eps, None, None, q, kp, table, pos, slot, page, fault)
        ops.gemm_heads(proj[:, :nq].unflatten(1, (H, dim)), w_uk, q.unflatten(1, (H, rank)))
        latent = torch.empty(n, H * rank, dtype=DT[dtype], device="cuda")
        ops.window_attention(q, proj[:, nq + rank:], latent, kp, kp[..., :rank], table, pos, slot, H, page, window, scale, None,
                             None, fault, step=_Step(pos, slot, decode_only=(n == 1 and i % 2 == 0)) if n != 2 else None,
                             gate_per_head=True)
        heads = torch.empty(n, H * vd, dtype=DT[dtype], device="cuda")
        ops.gemm_heads(latent.unflatten(1, (H, rank)), w_uv, heads.unflatten(1, (H, vd)))
        got[rows] = heads
    assert int(fault[0]) == 0
    stored = torch.stack([kp[int(perm[p // page]), 0, p % page] for p in range(L)])
    _close(stored, c, 2e-2 if dtype == "bfloat16" else 1e-5, "cache rows")
    _close(got, ref, 4e-2 if dtype == "bfloat16" else 1e-4, "windowed latent attention")


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n,d", [(37, 64), (5, 40), (130, 192), (1, 1000)])
def test_norm_behind_a_sublayer_activations_and_soft_cap(dtype, n, d):
    """``x += g_b * rms(update)`` and the norm of the sum in one kernel, the stream in 32-bit; the three activations of a
    feed-forward without a gate; the bound on the logits; the embedding's scale."""
    from tiny_inference_server_b200.kernels import ops
    torch.manual_seed(n + d)
    eps = 1e-5
    x = torch.randn(n, d) * 5.0
    y = (torch.randn(n, d) * 3.0).to(DT[dtype])
    g_b, g_n = 0.37, 1.4
    stream = x.clone().cuda()
    out = torch.empty(n, d, dtype=DT[dtype], device="cuda")
    ops.add_rmsnorm(stream, y.cuda(), torch.full((d,), g_n, device="cuda"), eps, out, kind="mean_eps",
                    delta_norm=(torch.full((d,), g_b, device="cuda"), eps, "mean_eps"))
    want = x.double() + plain.rms(y.double(), eps) * g_b
    _close(stream, want, 1e-6, "stream after a normed update")
    _close(out, plain.rms(want, eps) * g_n, 1e-2 if dtype == "bfloat16" else 1e-5, "norm of the sum")
    only_sum = x.clone().cuda()
    ops.add_rmsnorm(only_sum, y.cuda(), None, 0.0, None, delta_norm=(torch.full((d,), g_b, device="cuda"), eps, "mean_eps"))
    _close(only_sum, want, 1e-6, "a normed update without a norm of the sum")
    z = (torch.randn(n, d) * 2.0).to(DT[dtype])
    for kind, fn in plain.ACTIVATIONS.items():
        res = torch.empty(n, d, dtype=DT[dtype], device="cuda")
        ops.activation(z.cuda(), res, kind)
        _close(res, fn(z.double()), 1e-2 if dtype == "bfloat16" else 1e-5, kind)
    if dtype == "float32":
        lg = (torch.randn(n, d) * 40.0)
        _close(ops.softcap_f32(lg.clone().cuda(), 30.0), 30.0 * torch.tanh(lg.double() / 30.0), 1e-5, "soft cap")
    table = torch.randn(50, d).to(DT[dtype])
    toks = torch.randint(0, 50, (n,))
    rows = torch.empty(n, d, device="cuda")
    ops.embed_rows(table.cuda(), toks.to(torch.int32).cuda(), rows, 0.7)
    _close(rows, table.double()[toks] * 0.7, 1e-6, "scaled embedding")


@gpu
@pytest.mark.parametrize("kind", ["relu2", "gelu_tanh", "silu"])
@pytest.mark.parametrize("n,K,N", [(1, 256, 512), (8, 1536, 6144), (33, 512, 1096), (8, 3072, 12288), (200, 256, 512)])
def test_product_with_the_activation_in_its_epilogue(kind, n, K, N):
    """``act(a @ w)``: few rows take a weight-streaming product whose epilogue applies the activation to the 32-bit sums
    (no activation kernel is launched), many rows the product and then the activation kernel."""
    from tiny_inference_server_b200.kernels import ops
    torch.manual_seed(n + K)
    a = (torch.randn(n, K) * 0.5).to(torch.bfloat16)
    w = (torch.randn(K, N) / math.sqrt(K)).to(torch.bfloat16)
    before = dict(ops.calls)
    got = ops.gemm_act(a.cuda(), w.cuda(), kind)
    torch.cuda.synchronize()
    fused = sum(ops.calls[k] - before.get(k, 0) for k in ("gemm_skinny", "gemm_stream"))
    if (n, K) == (8, 1536):                              # a decode step's rows at a small model's sizes
        assert fused == 1, dict(ops.calls)
    if n > 64:
        assert fused == 0, dict(ops.calls)
    _close(got, plain.ACTIVATIONS[kind](a.double() @ w.double()), 1e-2, f"{kind} behind a product of {n} rows")


# ------------------------------------------------------------------------------------------------
# GPU: the whole model through the engine
# ------------------------------------------------------------------------------------------------

@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B1", "B2", "B3", "B4"])
@pytest.mark.parametrize("mode", ["whole", "tail", "chunks", "mixed"])
def test_replay_gpu(name, mode, dtype, tmp_path, tmp_path_factory):
    raw, page, folder, seqs, ref, _, _ = _setup(name, tmp_path_factory)
    steps = _steps(mode, seqs, max_live=3)
    runner, _ = _replay_and_compare(raw, page, folder, seqs, ref, steps, str(tmp_path / "out"), dtype, "cuda:0", TOL[dtype],
                                    max_live=3, poison=(mode == "mixed"), shuffle=(mode == "mixed"), outliers=BF16_OUTLIERS[dtype])
    if mode == "mixed" and name == "B1":          # its requests are long enough for the pool to turn over
        pool = runner.cache.groups[0].pool
        assert pool.allocations > pool.num_pages, "the trace does not use pages again"


@gpu
def test_layers_of_the_stream_gpu(tmp_path_factory):
    """The residual stream after every layer in float32 on the device against the plain layers."""
    raw, page, folder, seqs, _, c, W = _setup("B4", tmp_path_factory)
    toks = seqs["r2"]
    _, layers = plain.plain_forward(c, W, toks, return_layers=True)
    runner = make_runner(folder, "float32", 64, page_size=page, max_live=1, cuda_graphs=False)
    from tiny_inference_server_b200.engine.batch import StepEntry
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
        err = float((got.double().cpu() - want).abs().max() / want.abs().max())
        assert err < 1e-4, f"stream after layer {i} ({c['layers'][i]['type']}): {err}"


def random_configuration(seed):
    """A configuration drawn at random: layer order, head counts, widths, ranks, windows, constants, all of it."""
    import random
    rng = random.Random(seed)
    pick = rng.choice
    layers = []
    kinds = ["attention", "latent_attention", "hgrn2"]
    rng.shuffle(kinds)
    for kind in kinds + [pick(kinds) for _ in range(rng.randint(0, 3))]:
        if kind == "attention":
            kv = pick([1, 2, 3])
            mixer = _diff(kv * pick([1, 2, 4]), kv, pick([8, 16, 24, 32, 64]), pick([8, 16, 32, 48, 64, 96]),
                          diff=pick([0.1, 0.3, 0.5, 0.8]), temp=pick([None, (0.25, 48), (0.1, 1), (1.0, 17)]),
                          scale=pick([None, 0.2]))
        elif kind == "latent_attention":
            mixer = _latent(pick([1, 2, 4, 5, 8]), pick([8, 16, 32, 48]), pick([8, 16, 24, 64]), pick([12, 16, 32, 48, 80, 96, 160]),
                            window=pick([1, 3, 16, 50, 64, 130, 200, 1000]), scale=pick([None, 0.2]))
        else:
            mixer = _hgrn(pick([1, 2, 3, 4]), pick([8, 16, 32, 64, 128]), pick([8, 16, 32, 64, 96]))
        mlp = _ff(pick([24, 32, 64, 100, 256])) if rng.random() < 0.75 else None
        layers.append({"type": kind, "mixer": mixer, "mlp": mlp})
    cfg = dict(architecture="Biruvik", vocab=rng.randint(40, 300), width=pick([24, 32, 48, 64, 96, 128, 192]),
               norm={"eps": pick([1e-5, 1e-6])}, layers=layers)
    if rng.random() < 0.7:
        cfg["embedding"] = {"scale": pick([0.5, 1.0, 2.0, 8.0])}
    if rng.random() < 0.7:
        cfg["logit_softcap"] = pick([5.0, 25.0, 50.0])
    return cfg, pick([8, 16, 16, 32])


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", [1, 2, 3, 4, 5, 6, 7, 8])
def test_configurations_drawn_at_random(seed, dtype, tmp_path):
    """Whatever config.json says runs without a change of code: configurations drawn at random, a mixed batch of five
    requests (one of them long, past every window) through three slots over shuffled pages (``BF16_OUTLIERS``)."""
    raw, page = random_configuration(seed)
    folder = make_folder(raw, 100 + seed, str(tmp_path / "m"))
    c, W = plain.read_config(folder), plain.read_weights(folder)
    g = torch.Generator().manual_seed(seed)
    seqs = {f"r{i}": torch.randint(0, raw["vocab"], (n,), generator=g).tolist() for i, n in enumerate([1, 2, 45, 700, 130])}
    ref = {rid: plain.plain_forward(c, W, toks).numpy() for rid, toks in seqs.items()}
    steps = trace_tools.trace_mixed(seqs, max_live=3, prefill_sizes=(64, 2, 130, 17))
    _replay_and_compare(raw, page, folder, seqs, ref, steps, str(tmp_path / "out"), dtype, "cuda:0", TOL[dtype], max_live=3,
                        poison=True, shuffle=True, outliers=BF16_OUTLIERS[dtype])


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_two_slots_used_again_and_again(dtype, tmp_path, tmp_path_factory):
    """Eight requests through two state slots: a recurrent state that is not cleared when its slot is given to the next
    request shows in that request's first tokens."""
    raw, page, folder, seqs, ref, _, _ = _setup("B1", tmp_path_factory)
    steps = trace_tools.trace_mixed(seqs, max_live=2, prefill_sizes=(2, 7, 3, 2), skip_every=4)
    _replay_and_compare(raw, page, folder, seqs, ref, steps, str(tmp_path / "out"), dtype, "cuda:0", TOL[dtype], max_live=2,
                        poison=True, outliers=BF16_OUTLIERS[dtype])


@gpu
@pytest.mark.parametrize("name", ["B1", "B4"])
def test_long_decoding_float32(name, tmp_path, tmp_path_factory):
    """A short prompt, then 300 tokens one by one, replayed from a graph: the states carry what hundreds of decode steps
    wrote, every step's attention reads the whole cache or its window as it slides over decoded tokens, and the query
    temperature passes several of its steps."""
    raw, page, folder, _, _, c, W = _setup(name, tmp_path_factory)
    g = torch.Generator().manual_seed(9)
    toks = torch.randint(0, raw["vocab"], (305,), generator=g).tolist()
    ref = {"a": plain.plain_forward(c, W, toks).numpy()}
    steps = trace_tools.trace_tail({"a": toks}, tail=300)
    runner = make_runner(folder, "float32", 320, page_size=page, max_live=1, debug_poison=True)
    out_dir = str(tmp_path / "out")
    TraceReplayer(runner, out_dir).run(json.dumps(s) for s in steps)
    assert runner.cache.drained()
    assert runner.graphs is not None and runner.graphs.replays > 250
    got = trace_tools.gather(steps, out_dir, raw["vocab"])
    for p in range(len(toks)):
        assert rel_err(got["a"][p], ref["a"][p]) < TOL["float32"], f"position {p}"


@gpu
def test_generate_through_the_scheduler(tmp_path, tmp_path_factory):
    raw, page, folder, seqs, _, c, W = _setup("B3", tmp_path_factory)
    prompts = [seqs["r0"], seqs["r4"], seqs["r1"], seqs["r5"]]
    want = [plain_greedy(c, W, p, 10) for p in prompts]
    sp = SamplingParams(max_new_tokens=10, temperature=0.0, ignore_eos=True)
    for kw in (dict(max_batch=4, max_tokens_per_step=2048), dict(max_batch=2, max_tokens_per_step=9)):
        eng = Engine.from_folder(folder, EngineConfig(dtype="float32", page_size=page, num_pages=40, **kw))
        assert eng.generate(prompts, sp) == want
        assert eng.runner.cache.drained()
    eng = Engine.from_folder(folder, EngineConfig(dtype="bfloat16", page_size=page, num_pages=40, max_batch=4))
    out = eng.generate(prompts, sp)
    assert [len(o) for o in out] == [10] * 4 and eng.runner.cache.drained()


@gpu
def test_command_line_generation_with_chunking_and_preemption(tmp_path, tmp_path_factory):
    """Greedy tokens through ``python -m tiny_inference_server_b200.cli`` equal the plain implementation's: whole
    prompts; a token budget of five (portions beside decoding requests); and so few pages that requests are preempted
    and fed again from their first token (their recurrent states start from zero again)."""
    from test_cli import _cli, _ids
    raw, page, folder, seqs, _, c, W = _setup("B1", tmp_path_factory)
    new = 8
    prompts = [seqs["r0"], seqs["r6"], seqs["r1"]]
    want = [plain_greedy(c, W, p, new) for p in prompts]
    args = ["--model", folder, "--greedy", "--ignore-eos", "--dtype", "float32", "--max-new-tokens", new,
            "--tokens-per-block", page, "--json"]
    for p in prompts:
        args += ["--prompt-ids", _ids(p)]
    r = _cli(*args)
    assert r.returncode == 0, r.stderr
    assert json.loads(r.stdout.strip().splitlines()[-1])["outputs"] == want
    r = _cli(*args, "--max-tokens-per-step", 5, "--max-batch", 2)
    assert r.returncode == 0, r.stderr
    assert json.loads(r.stdout.strip().splitlines()[-1])["outputs"] == want
    g = torch.Generator().manual_seed(31)
    prompts = [torch.randint(0, raw["vocab"], (page - 1,), generator=g).tolist() for _ in range(4)]
    want = [plain_greedy(c, W, p, new) for p in prompts]
    args = ["--model", folder, "--greedy", "--ignore-eos", "--dtype", "float32", "--max-new-tokens", new,
            "--tokens-per-block", page, "--json", "--num-pages", 5, "--plan", "cur", "--max-batch", 4,
            "--max-tokens-per-step", 16]
    for p in prompts:
        args += ["--prompt-ids", _ids(p)]
    r = _cli(*args)
    assert r.returncode == 0, r.stderr
    out = json.loads(r.stdout.strip().splitlines()[-1])
    assert out["outputs"] == want
    assert out["stats"]["preempts"] > 0 and out["stats"]["replays"] > 0
