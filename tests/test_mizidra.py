"""The Mizidra architecture in the engine against the plain implementation (``plain_mizidra``): each mechanism
alone, whole prompts against token-by-token decoding, portions down to two tokens, mixed batches with pages and
state slots used again, a key far back and keys at page borders, memory far back through the recurrent states, the
first tokens of a sequence, long decoding, other sizes (also sizes that are equal or 1), and greedy generation
through ``Engine``.  Configurations and weights are made here; where random numbers would hide a fault the inputs
are planted so that it shows.

CPU tests run the engine with the PyTorch references in place of the kernels (``ref_ops``): they check the plumbing
(configuration, weights, cache, state, batch).  GPU tests run the CUDA kernels."""
import json
import math
import os

import numpy as np
import pytest
import torch

import plain_mizidra as plain
import trace_tools
from tiny_inference_server_b200.api import Engine, SamplingParams
from tiny_inference_server_b200.config import ConfigError, EngineConfig, MizidraConfig
from tiny_inference_server_b200.registry import build_model, config_from_dict, config_from_folder
from tiny_inference_server_b200.trace import TraceReplayer, make_runner

# ------------------------------------------------------------------------------------------------
# configurations: every size differs between them
# ------------------------------------------------------------------------------------------------


def _delta(heads, kv, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv}


def _latent(heads, dim, rot, vdim, rank, base=10000.0, scaling=None, scale=None, dims=None):
    r = {"base": base, "dims": dims or rot}
    if scaling:
        r["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": vdim, "kv_rank": rank, "rot": r,
            "scale": scale or (dim + rot) ** -0.5}


def _lightning(heads, dim, vdim, decay):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}


def _moe(experts, top, ff, groups=None, shared=None):
    r = {"experts": experts, "top": top}
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    f = {"kind": "moe", "expert": {"ff": ff}, "router": r}
    if shared:
        f["shared"] = {"ff": shared}
    return f


M1 = dict(architecture="Mizidra", vocab=131, width=64, norm={"eps": 1e-5}, layers=[
    {"type": "lightning", "mixer": _lightning(2, 16, 24, (0.9, 0.999)), "mlp": _moe(6, 3, 24, groups=(3, 2), shared=40)},
    {"type": "latent_attention", "mixer": _latent(4, 16, 8, 24, 40, scaling=(4.0, 64, 8.0, 1.0)), "mlp": None},
    {"type": "delta", "mixer": _delta(4, 2, 16, 8, 3), "mlp": _moe(6, 3, 24, groups=(3, 2), shared=40)},
    {"type": "latent_attention", "mixer": _latent(2, 8, 16, 16, 16, base=500.0, scale=0.3), "mlp": _moe(4, 2, 32)},
    {"type": "delta", "mixer": _delta(2, 2, 24, 40, 2), "mlp": None},
])
# sizes that are equal or 1 where M1's differ: one head, one kv head, one group, one chosen expert, one tap
M2 = dict(architecture="Mizidra", vocab=67, width=32, norm={"eps": 1e-6}, layers=[
    {"type": "delta", "mixer": _delta(1, 1, 16, 16, 1), "mlp": _moe(2, 1, 16, groups=(1, 1))},
    {"type": "latent_attention", "mixer": _latent(1, 16, 16, 16, 16, scaling=(2.0, 16, 4.0, 2.0)), "mlp": _moe(3, 1, 16, shared=16)},
    {"type": "lightning", "mixer": _lightning(1, 16, 16, (1.0,)), "mlp": None},
])
# sizes that fit no vector, tile or alignment: every kernel's plain path
M3 = dict(architecture="Mizidra", vocab=53, width=40, norm={"eps": 1e-6}, layers=[
    {"type": "latent_attention", "mixer": _latent(3, 10, 6, 7, 22, base=100.0, dims=4), "mlp": _moe(5, 2, 27, shared=13)},
    {"type": "lightning", "mixer": _lightning(3, 10, 6, (0.5, 0.8, 0.97)), "mlp": _moe(5, 2, 27)},
    {"type": "delta", "mixer": _delta(2, 1, 6, 10, 6), "mlp": None},
])
# sizes of the fast paths: the recurrences with a head's columns split over CTAs, attention on the tensor cores
M4 = dict(architecture="Mizidra", vocab=90, width=96, norm={"eps": 1e-6}, layers=[
    {"type": "delta", "mixer": _delta(4, 1, 32, 64, 4), "mlp": _moe(8, 4, 32, groups=(4, 2), shared=64)},
    {"type": "lightning", "mixer": _lightning(2, 64, 64, (0.95, 0.7)), "mlp": None},
    {"type": "latent_attention", "mixer": _latent(8, 32, 16, 32, 48, base=1e6, scaling=(8.0, 32, 16.0, 1.0)),
     "mlp": _moe(8, 4, 32, groups=(4, 2), shared=64)},
])
CONFIGS = {"M1": (M1, 16), "M2": (M2, 8), "M3": (M3, 12), "M4": (M4, 16)}
LENGTHS = {"M1": [1, 2, 3, 30, 75, 41, 9, 60], "M2": [1, 5, 40, 33, 17, 64], "M3": [2, 4, 50, 90, 23, 37],
           "M4": [3, 1, 45, 20, 70]}


def _spread(n):
    """n numbers in [0, 1] of which no two pairs have the same sum (greedily, the smallest integers that keep it so,
    divided by the largest): neither two experts nor two groups of experts weigh the same."""
    vals, sums, x = [], set(), 0
    while len(vals) < n:
        new = {x + v for v in vals} | {2 * x}
        if not (new & sums):
            vals.append(x)
            sums |= new
        x += 1
    return [v / max(vals[-1], 1) for v in vals]


def make_tensors(cfg, seed, calm_router=False):
    """Weights of a size that makes every mechanism matter: projections of unit gain (queries, keys and the router
    sharper), decays between nearly 0 and nearly 1, sinks and corrections of the order of the scores they meet;
    rounded to bfloat16 so that both precisions and the plain implementation hold the same numbers.
    ``calm_router``: the router's matrix is small and the corrections are spread so that neither two experts' choosing
    scores nor two groups' strengths are ever close — what the bfloat16 runs are compared on: there the rounding of a router's input would turn
    a close call the other way now and then, and a token that meets other experts differs by far more than rounding."""
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, spec in build_model(cfg).expected_tensors().items():
        shape = tuple(spec.shape)
        leaf = name.split(".", 1)[1] if name.startswith("l") else name
        rnd = torch.randn(shape, generator=gen)
        uni = torch.rand(shape, generator=gen)
        if name == "embed":
            t = rnd * 0.5
        elif leaf in ("norm1", "norm2", "mix.norm", "mix.dkv.norm") or name in ("final.norm", "embed.norm"):
            t = 1.0 + rnd * 0.2
        elif leaf.endswith(".conv"):
            t = rnd * 0.5
        elif leaf == "mix.A_log":
            t = -3.0 + 3.5 * uni
        elif leaf == "mix.dt_bias":
            t = -3.0 + 4.0 * uni
        elif leaf == "mix.sink":
            t = rnd * 1.5
        elif leaf == "mlp.correction" and calm_router:
            t = torch.tensor(_spread(shape[0]))[torch.randperm(shape[0], generator=gen)] * 1.5 - 1.2
        elif leaf == "mlp.router" and calm_router:
            t = rnd * 0.005 / math.sqrt(shape[1])
        elif leaf == "mlp.correction":
            t = rnd * 0.4 - 0.6                     # choosing scores on both sides of zero
        elif len(shape) == 2:
            gain = 2.0 if leaf in ("mix.q", "mix.k", "mix.dkv") else (4.0 if leaf == "mlp.router" else 1.0)
            t = rnd * gain / math.sqrt(shape[1])
        else:
            raise AssertionError(f"no rule for {name} {shape}")
        out[name] = t.to(torch.bfloat16).contiguous()
    return out


def make_folder(raw, seed, folder, calm_router=False):
    from safetensors.torch import save_file
    cfg = config_from_dict(json.loads(json.dumps(raw)))
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg.to_dict(), f)
    save_file(make_tensors(cfg, seed, calm_router), os.path.join(folder, "model.safetensors"))
    return folder


def closest_call(c, W, seqs):
    """The smallest margin by which any routing decision of the plain model on these sequences is taken: between the last
    kept and the first dropped group, and between the last chosen and the first not chosen expert."""
    margins = []
    inner = plain.route

    def spy(h, W_, p, router):
        E, top = router["experts"], router["top"]
        pick = torch.sigmoid(h @ W_[p + "router"].T) + W_[p + "correction"]
        g = router.get("groups")
        if g:
            per = pick.view(-1, g["count"], E // g["count"])
            strength = per.topk(min(2, E // g["count"]), dim=-1).values.sum(-1)
            order = strength.sort(-1, descending=True)
            if g["keep"] < g["count"]:
                margins.append(float((order.values[:, g["keep"] - 1] - order.values[:, g["keep"]]).min()))
            ok = torch.zeros_like(strength, dtype=torch.bool).scatter_(1, order.indices[:, :g["keep"]], True)
            pick = per.masked_fill(~ok[:, :, None], float("-inf")).reshape(-1, E)
        ranked = pick.sort(-1, descending=True).values
        if top < E:
            margins.append(float((ranked[:, top - 1] - ranked[:, top]).min()))
        return inner(h, W_, p, router)

    plain.route = spy
    try:
        for toks in seqs.values():
            plain.plain_forward(c, W, toks)
    finally:
        plain.route = inner
    return min(margins) if margins else float("inf")


_cache = {}


def _setup(name, tmp_path_factory, calm_router=False):
    key = name
    name = name.rstrip("c")
    if calm_router:
        key = name + "c"
    if key not in _cache:
        raw, page = CONFIGS[name]
        folder = make_folder(raw, 17 + ord(name[-1]), str(tmp_path_factory.mktemp(f"mizidra{key}")), calm_router)
        c, W = plain.read_config(folder), plain.read_weights(folder)
        g = torch.Generator().manual_seed(5)
        seqs = {f"r{i}": torch.randint(0, raw["vocab"], (n,), generator=g).tolist() for i, n in enumerate(LENGTHS[name])}
        ref = {rid: plain.plain_forward(c, W, toks).numpy() for rid, toks in seqs.items()}
        if calm_router:
            assert closest_call(c, W, seqs) > 0.002, "the weights made for bfloat16 have a close routing decision"
        _cache[key] = (raw, page, folder, seqs, ref, c, W)
    return _cache[key]


def rel_err(got, ref):
    """Difference of two rows of logits, mean taken off, root mean square, over that of the reference."""
    d = np.asarray(got, dtype=np.float64) - ref
    d = d - d.mean()
    r = ref - ref.mean()
    return float(np.sqrt((d * d).mean()) / max(np.sqrt((r * r).mean()), 1e-9))


TOL = {"float32": 2e-4, "bfloat16": 6e-2}
#: In float32 every position agrees.  In bfloat16 one position in a hundred may differ by more than the tolerance (by less
#: than 1): among hundreds of positions of random weights a few are ill-conditioned (a norm of a nearly vanishing
#: read-out), and there rounding the activations between kernels — done in plain arithmetic on the CPU, at the same
#: places — moves the logits as far as the kernels do.
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
    folder = make_folder(M1, 1, str(tmp_path / "m"))
    cfg = config_from_folder(folder)
    assert isinstance(cfg, MizidraConfig)
    again = config_from_dict(cfg.to_dict())
    assert again.to_dict() == cfg.to_dict()
    names = set(build_model(cfg).expected_tensors())
    assert {"embed", "embed.norm", "final.norm", "head", "l0.mix.norm", "l0.mlp.e5.down", "l0.mlp.shared.sg",
            "l0.mlp.correction", "l1.mix.dkv.norm", "l1.mix.sink", "l1.mix.uk", "l2.mix.q.conv", "l2.mix.A_log",
            "l2.mix.a"} <= names
    assert "l1.norm2" not in names and "l3.mlp.shared.gate" not in names and "l0.mix.q.conv" not in names
    shapes = {n: tuple(s.shape) for n, s in build_model(cfg).expected_tensors().items()}
    assert shapes["l1.mix.q"] == (4 * 24, 64) and shapes["l1.mix.dkv"] == (48, 64) and shapes["l1.mix.uv"] == (96, 40)
    assert shapes["l2.mix.k"] == (32, 64) and shapes["l2.mix.v"] == (32, 64) and shapes["l0.mix.norm"] == (48,)


def test_config_errors_name_the_problem():
    def broken(change):
        bad = json.loads(json.dumps(M1))
        change(bad)
        return bad

    with pytest.raises(ConfigError, match="layers\\[0\\].type"):
        config_from_dict(broken(lambda c: c["layers"][0].update(type="conv_only")))
    with pytest.raises(ConfigError, match="not a multiple"):
        config_from_dict(broken(lambda c: c["layers"][2]["mixer"].update(heads=3)))
    with pytest.raises(ConfigError, match="one number per head"):
        config_from_dict(broken(lambda c: c["layers"][0]["mixer"].update(decay=[0.5])))
    with pytest.raises(ConfigError, match="exceeds"):
        config_from_dict(broken(lambda c: c["layers"][0]["mlp"]["router"].update(top=5)))
    with pytest.raises(ConfigError, match="rot.dims"):
        config_from_dict(broken(lambda c: c["layers"][1]["mixer"]["rot"].update(dims=10)))
    with pytest.raises(ConfigError, match="missing keys: width"):
        config_from_dict(broken(lambda c: c.pop("width")))


@pytest.mark.parametrize("rot,base,scaling", [(8, 10000.0, None), (8, 10000.0, (4.0, 64, 8.0, 1.0)), (32, 1e6, (8.0, 512, 32.0, 1.0)),
                                              (16, 50.0, (2.0, 16, 4.0, 2.0)), (6, 100.0, (16.0, 4096, 1.0, 0.01))])
def test_rotation_tables(rot, base, scaling):
    """The engine's tables against the plain frequencies, also where the blend's ends are clamped to the first and the
    last channel."""
    from tiny_inference_server_b200.parts.positions import RotaryRescaled
    sc = dict(zip(("factor", "original", "fast", "slow"), scaling)) if scaling else None
    f, mag = plain.rotary_frequencies({"dims": rot, "base": base, "scaling": sc})
    cos, sin = RotaryRescaled(rot, base, 300, scaling=sc).tables()
    ang = torch.arange(300, dtype=torch.float64)[:, None] * f[None, :]
    assert float((cos.double() - torch.cos(ang) * mag).abs().max()) < 1e-6
    assert float((sin.double() - torch.sin(ang) * mag).abs().max()) < 1e-6
    if scaling:
        plain_f, _ = plain.rotary_frequencies({"dims": rot, "base": base})
        assert mag > 1.0 and bool((f <= plain_f).all())
        assert float((f - plain_f).abs().max()) > 0 or rot == 6       # the last case blends nothing: its ramp starts past the last channel


# ------------------------------------------------------------------------------------------------
# the engine's plumbing on the CPU
# ------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("name", ["M1", "M2", "M3", "M4"])
@pytest.mark.parametrize("mode", ["whole", "tail", "chunks", "mixed"])
def test_replay_cpu(name, mode, tmp_path, tmp_path_factory, ref_ops):
    raw, page, folder, seqs, ref, _, _ = _setup(name, tmp_path_factory)
    steps = _steps(mode, seqs, max_live=3)
    _replay_and_compare(raw, page, folder, seqs, ref, steps, str(tmp_path / "out"), "float32", "cpu", 1e-4, max_live=3,
                        poison=(mode == "mixed"))


def plain_greedy(c, W, prompt, new):
    ids = list(prompt)
    for _ in range(new):
        ids.append(int(plain.plain_forward(c, W, ids)[-1].argmax()))
    return ids[len(prompt):]


def test_generate_cpu(tmp_path, tmp_path_factory, ref_ops):
    raw, page, folder, seqs, ref, c, W = _setup("M2", tmp_path_factory)
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


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,kd,vd", [(4, 2, 16, 8), (2, 2, 24, 40), (3, 1, 32, 64), (1, 1, 128, 96), (2, 1, 12, 20)])
def test_delta_rule_with_a_decay_per_head(dtype, H, G, kd, vd):
    """The recurrence over portions of 1..70 rows equals the token-by-token rule on the whole sequence.  Head 0
    hardly decays and is written strongly at position 1 only: its read-out 250 tokens later still is that value."""
    from tiny_inference_server_b200.kernels import ops
    torch.manual_seed(kd + vd)
    L = 260
    nq, nv = G * kd, H * vd
    qkv = torch.randn(L, 2 * nq + nv)
    beta = torch.randn(L, H)
    a = torch.randn(L, H)
    a_log = -1.0 + torch.rand(H)
    dt_bias = -1.0 + torch.rand(H)
    a_log[0] = -12.0                                       # head 0: decay of nearly 1
    beta[:, 0] = -20.0                                     # ... and no writes
    beta[1, 0] = 20.0                                      # but one
    mark = torch.randn(kd)
    qkv[1, nq:nq + kd] = mark                              # its key (q/k head 0) ...
    qkv[L - 3, :kd] = mark                                 # ... asked for again near the end
    gate = torch.randn(L, nv)
    norm_w = 1 + 0.2 * torch.randn(vd)
    eps = 1e-5
    cast = lambda t: t.to(DT[dtype])
    qkv, beta, a, gate = cast(qkv), cast(beta), cast(a), cast(gate)
    q = qkv[:, :nq].double().view(L, G, kd)
    k = qkv[:, nq:2 * nq].double().view(L, G, kd)
    v = qkv[:, 2 * nq:].double().view(L, H, vd)
    q = (q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * kd ** -0.5).repeat_interleave(H // G, dim=1)
    k = (k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)).repeat_interleave(H // G, dim=1)
    decay = torch.exp(-torch.exp(a_log.double()) * torch.nn.functional.softplus(a.double() + dt_bias.double()))
    b = torch.sigmoid(beta.double())
    S = torch.zeros(H, kd, vd, dtype=torch.float64)
    o = torch.zeros(L, H, vd, dtype=torch.float64)
    for t in range(L):
        S = decay[t][:, None, None] * S
        u = b[t][:, None] * (v[t] - torch.einsum("hdv,hd->hv", S, k[t]))
        S = S + k[t][:, :, None] * u[:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    raw_far = o[L - 3, 0].clone()
    ref = (plain.rms(o, eps) * norm_w.double() * plain.silu(gate.double().view(L, H, vd))).reshape(L, nv)
    want_far = v[1, 0] * kd ** -0.5
    assert float((raw_far - want_far).abs().max()) < 0.05 * float(want_far.abs().max())
    state = torch.zeros(3, H * kd * vd + 11, device="cuda")
    got = torch.zeros(L, nv, dtype=DT[dtype], device="cuda")
    fed, i = 0, 0
    cuts = [1, 2, 17, 1, 33, 70, 2, 16, 5]
    while fed < L:
        n = min(cuts[i % len(cuts)], L - fed)
        i += 1
        rows = slice(fed, fed + n)
        row_slot, row_last = _rows([n], [2])
        out = torch.empty(n, nv, dtype=DT[dtype], device="cuda")
        ops.delta_rule(qkv[rows].cuda(), beta[rows].cuda(), a[rows].cuda(), gate[rows].cuda(), a_log.cuda(), dt_bias.cuda(),
                       norm_w.cuda(), eps, 1e-6, kd ** -0.5, state, out, row_slot, row_last, H, G, kd, vd,
                       requests=1 if i % 2 else None, decay_per_head=True, gate_act="silu")
        got[rows] = out
        fed += n
    _close(got, ref, 3e-2 if dtype == "bfloat16" else 1e-4, "delta rule")
    _close(state[2, :H * kd * vd], S.reshape(-1), 1e-4, "state")
    assert float(state[0].abs().max()) == 0 and float(state[2, H * kd * vd:].abs().max()) == 0


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,kd,vd", [(2, 16, 24), (1, 16, 16), (3, 10, 6), (2, 64, 64), (1, 128, 32), (4, 32, 96)])
def test_linear_attention_in_portions_and_far_memory(dtype, H, kd, vd):
    """Two sequences side by side in slots 2 and 0, in portions of 1..70 rows, equal the token-by-token rule.  Head 0
    does not decay at all: what position 1 wrote (a key ten times the usual size) is what a query along that key reads
    250 tokens later; the last head forgets within a few tokens."""
    from tiny_inference_server_b200.kernels import ops
    torch.manual_seed(kd * 3 + vd)
    L = 260
    nq, nv = H * kd, H * vd
    decay = torch.tensor([1.0] + [0.97] * (H - 2) + ([0.4] if H > 1 else []))
    seqs = []
    for s in range(2):
        qkv = torch.randn(L, 2 * nq + nv) * 0.5
        qkv[:, nq:nq + kd] *= 0.05                         # head 0 writes little, but for one token
        mark = torch.randn(kd).abs() + 1.0                 # positive: silu keeps it
        qkv[1, nq:nq + kd] = mark * 10.0
        qkv[L - 3, :kd] = mark * 10.0
        seqs.append((qkv.to(DT[dtype]), torch.randn(L, nv).to(DT[dtype])))
    norm_w = 1 + 0.2 * torch.randn(nv)
    eps = 1e-5
    refs, finals = [], []
    for qkv, gate in seqs:
        q = plain.silu(qkv[:, :nq].double()).view(L, H, kd)
        k = plain.silu(qkv[:, nq:2 * nq].double()).view(L, H, kd)
        v = plain.silu(qkv[:, 2 * nq:].double()).view(L, H, vd)
        S = torch.zeros(H, kd, vd, dtype=torch.float64)
        o = torch.zeros(L, H, vd, dtype=torch.float64)
        for t in range(L):
            S = decay.double()[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
            o[t] = torch.einsum("hdv,hd->hv", S, q[t])
        # the far write dominates the read-out of head 0 at L - 3
        far = (k[1, 0] @ q[L - 3, 0]) * v[1, 0]
        assert float((o[L - 3, 0] - far).abs().max()) < 0.35 * float(far.abs().max())
        refs.append(plain.nrm(o.reshape(L, nv), norm_w.double(), eps) * torch.sigmoid(gate.double()))
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
        qkv = torch.cat([seqs[s][0][fed[s]:fed[s] + c] for s, c in parts]).cuda()
        gate = torch.cat([seqs[s][1][fed[s]:fed[s] + c] for s, c in parts]).cuda()
        row_slot, row_last = _rows([c for _, c in parts], [(2, 0)[s] for s, _ in parts])
        out = torch.empty(qkv.shape[0], nv, dtype=DT[dtype], device="cuda")
        ops.linear_attention(qkv, gate, decay.cuda(), norm_w.cuda(), eps, state, out, row_slot, row_last, H, kd, vd,
                             requests=len(parts) if i % 2 else None)
        at = 0
        for s, c in parts:
            got[s][fed[s]:fed[s] + c] = out[at:at + c]
            at += c
            fed[s] += c
    for s in range(2):
        _close(got[s], refs[s], 3e-2 if dtype == "bfloat16" else 1e-4, "linear attention")
        _close(state[(2, 0)[s], :nq * vd], finals[s], 2e-2 if dtype == "bfloat16" else 1e-4, "state")
    assert float(state[1].abs().max()) == 0


class _Step:
    """What an attention kernel asks of a step, for one request's portion outside the engine."""

    def __init__(self, positions, row_slot, decode_only=False):
        self.positions, self.row_slot, self.decode_only = positions, row_slot, decode_only
        self.max_position = int(positions.max())

    def plan(self, planner):
        return planner.infer(self.positions, self.row_slot)


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,flat,rot,rank,page,dims", [(4, 16, 8, 40, 16, 8), (2, 8, 16, 16, 4, 12), (3, 10, 6, 22, 12, 2),
                                                       (8, 32, 16, 48, 16, 16), (1, 16, 16, 16, 8, 16), (16, 8, 32, 96, 16, 32)])
def test_latent_cache_sink_and_a_key_far_back(dtype, H, flat, rot, rank, page, dims):
    """The step between the projections and the cache (norm of the compressed vector, rotation of the shared key
    slice and of the queries' slices) and attention with a sink over that cache, in portions and single rows over
    scattered pages.  Rows near the end ask for key 3, several hundred keys back, and for the keys at the last and
    first place of a page; one head's sink is so large that it takes most of the weight."""
    from tiny_inference_server_b200.kernels import ops
    from tiny_inference_server_b200.parts.positions import RotaryRescaled
    torch.manual_seed(H * 10 + rank)
    L = 333
    qd, row = flat + rot, rank + rot
    rot_cfg = {"dims": dims, "base": 1000.0, "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}}
    proj = torch.randn(L, H * qd + row + 3)                # three columns of padding behind
    dkv_at = H * qd
    sink = torch.randn(H)
    sink[H - 1] = 6.0
    cw = 1 + 0.2 * torch.randn(rank)
    eps, scale = 1e-5, 0.7 * row ** -0.5
    proj = proj.to(DT[dtype])
    pos_all = torch.arange(L)
    # plain: the cache rows and the queries as the attention meets them
    low = proj[:, dkv_at:dkv_at + row].double()
    c = plain.nrm(low[:, :rank], cw.double(), eps)
    k_rot = plain.rotate(low[:, rank:], pos_all, rot_cfg)
    q = proj[:, :dkv_at].double().view(L, H, qd)
    q_flat = torch.randn(L, H, rank, dtype=torch.float64)   # stands for the queries' unrotated part after its product
    asked = {L - 1: 3, L - 2: page - 1, L - 5: 2 * page, L - 40: 3}
    for r_, j in asked.items():                             # head 0 of these rows looks along the latent of key j
        q_flat[r_, 0] = c[j] * 12.0 / scale / float(c[j] @ c[j])
    q_rot = plain.rotate(q[..., flat:], pos_all, rot_cfg)
    q_flat = q_flat.to(DT[dtype]).double()
    rows_k = torch.cat([c, k_rot], dim=-1)
    q_all = torch.cat([q_flat, q_rot], dim=-1)
    if dtype == "bfloat16":
        rows_k, q_all = rows_k.to(torch.bfloat16).double(), q_all.to(torch.bfloat16).double()
    k_all = rows_k[:, None, :].expand(L, H, row)
    ref = plain.attend_with_sink(q_all, k_all, k_all[..., :rank], scale, sink.double()).reshape(L, H * rank)
    without = plain.attend_with_sink(q_all, k_all, k_all[..., :rank], scale, None).reshape(L, H * rank)
    for r_, j in asked.items():                             # the asked key carries the row
        w = torch.softmax(torch.cat([(q_all[r_, 0] @ rows_k[:r_ + 1].T) * scale, sink[:1].double()]), 0)
        assert float(w[j]) > 0.5, (r_, j, float(w[j]))
    assert float((ref - without).abs().max()) > 0.2         # the sink matters
    n_pages = (L + page - 1) // page + 3
    kp = torch.full((n_pages, 1, page, row), 1e4, dtype=DT[dtype], device="cuda")
    perm = torch.randperm(n_pages)[: (L + page - 1) // page].to(torch.int32)
    table = torch.full((3, len(perm) + 2), -1, dtype=torch.int32)
    table[1, :len(perm)] = perm
    table = table.cuda()
    fault = torch.zeros(4, dtype=torch.int32, device="cuda")
    cos, sin = (t.cuda() for t in RotaryRescaled(rot, 1000.0, 512, scaling=rot_cfg["scaling"], rotary_dim=dims).tables())
    got = torch.zeros(L, H * rank, dtype=DT[dtype], device="cuda")
    fed, i = 0, 0
    cuts = [5, 2, 1, 1, 30, 2, 64, 100]
    while fed < L:
        n = min(cuts[i % len(cuts)], max(1, L - 4 - fed)) if fed < L - 4 else 1      # the last four rows alone
        i += 1
        rows = slice(fed, fed + n)
        pos = torch.arange(fed, fed + n, dtype=torch.int32, device="cuda")
        slot = torch.full((n,), 1, dtype=torch.int32, device="cuda")
        qbuf = torch.zeros(n, H * row, dtype=DT[dtype], device="cuda")
        ops.latent_prepare(proj[rows].cuda(), dkv_at, H, flat, rot, rank, cw.cuda(), eps, cos, sin, qbuf, kp, table, pos,
                           slot, page, fault)
        _close(qbuf.view(n, H, row)[:, :, rank:], q_rot[rows], 2e-2 if dtype == "bfloat16" else 1e-5, "rotated queries")
        qbuf.view(n, H, row)[:, :, :rank] = q_flat[rows].to(DT[dtype]).cuda()
        out = torch.empty(n, H * rank, dtype=DT[dtype], device="cuda")
        ops.window_attention(qbuf, None, out, kp, kp[..., :rank], table, pos, slot, H, page, None, scale, None, None, fault,
                             step=_Step(pos, slot, decode_only=(n == 1 and i % 2 == 0)) if n != 2 else None, sink=sink.cuda())
        got[rows] = out
        fed += n
    assert int(fault[0]) == 0
    stored = torch.stack([kp[int(perm[p // page]), 0, p % page] for p in range(L)])
    _close(stored, rows_k, 2e-2 if dtype == "bfloat16" else 1e-5, "cache rows")
    _close(got, ref, 4e-2 if dtype == "bfloat16" else 1e-4, "attention with a sink")


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_products_per_head(dtype):
    from tiny_inference_server_b200.kernels import ops
    torch.manual_seed(3)
    n, H, K, N = 37, 5, 24, 40
    a = torch.randn(n, H * (K + 8)).to(DT[dtype]).cuda()
    w = (torch.randn(H, K, N) / math.sqrt(K)).to(DT[dtype]).cuda()
    out = torch.zeros(n, H * (N + 16), dtype=DT[dtype], device="cuda")
    a_v = a.view(n, H, K + 8)[:, :, :K]
    ops.gemm_heads(a_v, w, out.view(n, H, N + 16)[:, :, :N])
    ref = torch.einsum("nhk,hkj->nhj", a_v.double().cpu(), w.double().cpu())
    _close(out.view(n, H, N + 16)[:, :, :N], ref, 1e-2 if dtype == "bfloat16" else 1e-5, "products per head")
    assert float(out.view(n, H, N + 16)[:, :, N:].abs().max()) == 0


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("E,top,groups,shared", [(8, 3, (2, 1), True), (6, 3, (3, 2), True), (5, 2, None, False), (2, 1, (1, 1), False),
                                                 (16, 6, (4, 2), True), (12, 2, (12, 3), False), (3, 3, None, True)])
def test_router_and_experts(dtype, E, top, groups, shared):
    """The router against the plain one on rows whose choosing scores are all negative (a group that is out of the
    race counts as minus infinity, not as zero), then the experts' products and the weighted sum."""
    from tiny_inference_server_b200.kernels import ops
    torch.manual_seed(E * 7 + top)
    n, d, F, SF = 45, 36, 22, 18
    p = "m."
    W = {p + "router": torch.randn(E, d) * 3.0 / math.sqrt(d), p + "correction": torch.randn(E) * 0.3 - 2.5,
         p + "shared.sg": torch.randn(1, d) / math.sqrt(d)}
    for e in range(E):
        W[f"{p}e{e}.gate"], W[f"{p}e{e}.up"] = torch.randn(F, d) / math.sqrt(d), torch.randn(F, d) / math.sqrt(d)
        W[f"{p}e{e}.down"] = torch.randn(d, F) / math.sqrt(F)
    W = {k: v.to(torch.bfloat16).double() for k, v in W.items()}
    x = torch.randn(n, d).to(DT[dtype])
    router = {"experts": E, "top": top}
    if groups:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    idx, w = plain.route(x.double(), W, p, router)
    assert float((torch.sigmoid(x.double() @ W[p + "router"].T) + W[p + "correction"]).max()) < 0   # all negative
    f32 = lambda t: t.float().cuda().contiguous()
    chosen, weights, sgate = ops.moe_route(x.cuda(), f32(W[p + "router"]), f32(W[p + "correction"]),
                                           f32(W[p + "shared.sg"]).reshape(-1) if shared else None,
                                           groups[0] if groups else 0, groups[1] if groups else 0, top)
    order_ref = idx.sort(-1)
    order_got = chosen.long().cpu().sort(-1)
    assert torch.equal(order_got.values, order_ref.values), "another choice of experts"
    _close(weights.cpu().gather(1, order_got.indices), w.gather(1, order_ref.indices), 1e-5, "weights")
    assert float((weights.sum(-1) - 1).abs().max()) < 1e-5
    if shared:
        _close(sgate, torch.sigmoid(x.double() @ W[p + "shared.sg"].T)[:, 0], 1e-5, "shared gate")
    cdt = lambda t: t.to(DT[dtype]).cuda().contiguous()
    w_gu = cdt(torch.stack([torch.stack([W[f"{p}e{e}.gate"], W[f"{p}e{e}.up"]]) for e in range(E)]))
    w_dn = cdt(torch.stack([W[f"{p}e{e}.down"] for e in range(E)]))
    hidden = ops.moe_gate_up(x.cuda(), chosen, w_gu)
    extra = torch.randn(n, d).to(DT[dtype])
    out = ops.moe_down(hidden, chosen, weights, w_dn, extra.cuda() if shared else None, sgate)
    ref = torch.zeros(n, d, dtype=torch.float64)
    for r in range(n):
        for k in range(top):
            ref[r] += w[r, k] * plain.gated_unit(x[r:r + 1].double(), W, f"{p}e{int(idx[r, k])}.")[0]
    if shared:
        ref += torch.sigmoid(x.double() @ W[p + "shared.sg"].T) * extra.double()
    _close(out, ref, 3e-2 if dtype == "bfloat16" else 1e-5, "experts")


@gpu
@pytest.mark.parametrize("n,d,F,E,top", [(300, 64, 96, 6, 3), (40, 96, 32, 16, 3), (1000, 32, 160, 3, 1), (129, 128, 64, 8, 8),
                                         (700, 128, 192, 6, 3), (400, 64, 64, 16, 3), (1024, 256, 128, 4, 2), (2048, 320, 448, 16, 1)])
def test_experts_of_many_rows(n, d, F, E, top):
    """Many bfloat16 rows: sorted by expert on the device, tiles on the tensor cores (``mma.sync`` tiles of 64 rows; from
    1024 pairs, with widths that are multiples of 64, ``tcgen05`` tiles of 128 rows).  Experts that no row chose, experts
    whose rows end in the middle of a tile, hidden sizes that end in the middle of a tile of columns; beside the kernels
    that take the same rows one dot product at a time."""
    from tiny_inference_server_b200.kernels import ops
    torch.manual_seed(n + E)
    p = "m."
    W = {}
    for e in range(E):
        W[f"{p}e{e}.gate"], W[f"{p}e{e}.up"] = torch.randn(F, d) / math.sqrt(d), torch.randn(F, d) / math.sqrt(d)
        W[f"{p}e{e}.down"] = torch.randn(d, F) / math.sqrt(F)
    W = {k: v.to(torch.bfloat16).double() for k, v in W.items()}
    x = torch.randn(n, d).to(torch.bfloat16)
    scores = torch.rand(n, E)
    if E == 16:
        scores[:, 5:9] = -1.0                                  # experts 5..8 get no row
    chosen = scores.topk(top, dim=-1).indices.to(torch.int32)
    weights = torch.rand(n, top)
    extra, sgate = torch.randn(n, d).to(torch.bfloat16), torch.rand(n)
    cdt = lambda t: t.to(torch.bfloat16).cuda().contiguous()
    w_gu = cdt(torch.stack([torch.stack([W[f"{p}e{e}.gate"], W[f"{p}e{e}.up"]]) for e in range(E)]))
    w_dn = cdt(torch.stack([W[f"{p}e{e}.down"] for e in range(E)]))
    before = ops.calls["moe_grouped"], ops.calls["moe_grouped_tc"]
    out = ops.moe_experts(x.cuda(), chosen.cuda(), weights.cuda(), w_gu, w_dn, extra.cuda(), sgate.cuda())
    big = n * top >= 1024 and d % 64 == 0 and F % 64 == 0
    assert (ops.calls["moe_grouped"], ops.calls["moe_grouped_tc"]) == (before[0] + (not big), before[1] + big)
    assert int(ops.tc_fault()[0]) == 0
    one_by_one = ops.moe_down(ops.moe_gate_up(x.cuda(), chosen.cuda(), w_gu), chosen.cuda(), weights.cuda(), w_dn, extra.cuda(),
                              sgate.cuda())
    ref = sgate.double()[:, None] * extra.double()
    for e in range(E):
        share = (weights.double() * (chosen == e)).sum(-1, keepdim=True)
        ref += share * plain.gated_unit(x.double(), W, f"{p}e{e}.")
    _close(out, ref, 3e-2, "experts, many rows")
    _close(one_by_one, ref, 3e-2, "experts, row by row")


# ------------------------------------------------------------------------------------------------
# GPU: the whole model through the engine
# ------------------------------------------------------------------------------------------------

@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["M1", "M2", "M3", "M4"])
@pytest.mark.parametrize("mode", ["whole", "tail", "chunks", "mixed"])
def test_replay_gpu(name, mode, dtype, tmp_path, tmp_path_factory):
    raw, page, folder, seqs, ref, _, _ = _setup(name, tmp_path_factory, calm_router=(dtype == "bfloat16"))
    steps = _steps(mode, seqs, max_live=3)
    runner, _ = _replay_and_compare(raw, page, folder, seqs, ref, steps, str(tmp_path / "out"), dtype, "cuda:0", TOL[dtype],
                                    max_live=3, poison=(mode == "mixed"), shuffle=(mode == "mixed"), outliers=BF16_OUTLIERS[dtype])
    if mode == "mixed" and name == "M1":          # its requests are long enough for the pool to turn over
        pool = runner.cache.groups[0].pool
        assert pool.allocations > pool.num_pages, "the trace does not use pages again"


def random_configuration(seed):
    """A configuration drawn at random: layer order, head counts, widths, taps, ranks, rotation, groups, all of it."""
    import random
    rng = random.Random(seed)
    pick = rng.choice
    layers = []
    kinds = ["delta", "latent_attention", "lightning"]
    rng.shuffle(kinds)
    for kind in kinds + [pick(kinds) for _ in range(rng.randint(0, 2))]:
        if kind == "delta":
            kv = pick([1, 2, 3])
            mixer = _delta(kv * pick([1, 2]), kv, pick([8, 16, 24, 32, 64]), pick([8, 16, 32, 64, 96]), pick([2, 3, 4, 5]))
        elif kind == "latent_attention":
            rot = pick([4, 8, 16, 32])
            scaling = pick([None, (pick([2.0, 8.0, 32.0]), pick([16, 64, 256]), pick([8.0, 32.0]), pick([1.0, 2.0]))])
            mixer = _latent(pick([1, 2, 4, 5, 8]), pick([8, 16, 32, 48]), rot, pick([8, 16, 24, 64]), pick([12, 16, 32, 48, 80, 96]),
                            base=pick([100.0, 10000.0, 1e6]), scaling=scaling, scale=pick([None, 0.2]),
                            dims=pick([rot, rot, max(2, rot // 2)]))
        else:
            heads = pick([1, 2, 3, 4])
            mixer = _lightning(heads, pick([8, 16, 32, 64]), pick([8, 16, 32, 64]), [rng.uniform(0.6, 1.0) for _ in range(heads)])
        mlp = None
        if rng.random() < 0.75:
            groups = pick([None, (2, 1), (2, 2), (3, 2), (4, 2)])
            per = pick([1, 2, 3, 4])
            experts = (groups[0] if groups else pick([1, 2, 3])) * per
            allowed = per * groups[1] if groups else experts
            mlp = _moe(experts, rng.randint(1, min(allowed, 6)), pick([8, 16, 24, 32, 64]), groups=groups,
                       shared=pick([None, 16, 40]))
        layers.append({"type": kind, "mixer": mixer, "mlp": mlp})
    return dict(architecture="Mizidra", vocab=rng.randint(40, 300), width=pick([24, 32, 48, 64, 96, 128]),
                norm={"eps": pick([1e-5, 1e-6])}, layers=layers), pick([8, 16, 16, 32])


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", [1, 2, 3, 4, 5, 6])
def test_configurations_drawn_at_random(seed, dtype, tmp_path):
    """Whatever config.json says runs without a change of code: six configurations drawn at random, a mixed batch of
    five requests (one of them long) through three slots over shuffled pages (``BF16_OUTLIERS``)."""
    raw, page = random_configuration(seed)
    folder = make_folder(raw, 100 + seed, str(tmp_path / "m"), calm_router=(dtype == "bfloat16"))
    c, W = plain.read_config(folder), plain.read_weights(folder)
    g = torch.Generator().manual_seed(seed)
    seqs = {f"r{i}": torch.randint(0, raw["vocab"], (n,), generator=g).tolist() for i, n in enumerate([1, 2, 45, 700, 130])}
    ref = {rid: plain.plain_forward(c, W, toks).numpy() for rid, toks in seqs.items()}
    if dtype == "bfloat16":
        assert closest_call(c, W, seqs) > 0.002, "the weights made for bfloat16 have a close routing decision"
    steps = trace_tools.trace_mixed(seqs, max_live=3, prefill_sizes=(64, 2, 130, 17))
    _replay_and_compare(raw, page, folder, seqs, ref, steps, str(tmp_path / "out"), dtype, "cuda:0", TOL[dtype], max_live=3,
                        poison=True, shuffle=True, outliers=BF16_OUTLIERS[dtype])


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_two_slots_used_again_and_again(dtype, tmp_path, tmp_path_factory):
    """Eight requests through two state slots: a state that is not cleared, or a slot's convolution history that
    leaks into the next request, shows in the first tokens of the later requests."""
    raw, page, folder, seqs, ref, _, _ = _setup("M1", tmp_path_factory, calm_router=(dtype == "bfloat16"))
    steps = trace_tools.trace_mixed(seqs, max_live=2, prefill_sizes=(2, 7, 3, 2), skip_every=4)
    _replay_and_compare(raw, page, folder, seqs, ref, steps, str(tmp_path / "out"), dtype, "cuda:0", TOL[dtype], max_live=2,
                        poison=True, outliers=BF16_OUTLIERS[dtype])


@gpu
@pytest.mark.parametrize("name", ["M1", "M4"])
def test_long_decoding_float32(name, tmp_path, tmp_path_factory):
    """A short prompt, then 300 tokens one by one, replayed from a graph: the states carry what hundreds of decode
    steps wrote, and every step's attention reads the whole cache."""
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
    raw, page, folder, seqs, _, c, W = _setup("M3", tmp_path_factory)
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
    and fed again from their first token (their recurrent states and convolution histories start from zero again)."""
    from test_cli import _cli, _ids
    raw, page, folder, seqs, _, c, W = _setup("M1", tmp_path_factory)
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
