"""The Kefisun architecture in the engine against the plain implementation (``plain_kefisun``): each
mechanism alone, whole prompts against token-by-token decoding, portions down to two tokens, mixed
batches with pages and state slots used again, keys at page borders and at the edge of the window,
memory far back through the recurrent state, the first tokens of a sequence, long decoding, and greedy
generation through ``Engine``.  Configurations and weights are made here; where random numbers would
hide a fault the inputs are planted so that it shows.

CPU tests run the engine with the PyTorch references in place of the kernels (``ref_ops``): they check
the plumbing (configuration, weights, cache, state, batch).  GPU tests run the CUDA kernels."""
import json
import math
import os

import numpy as np
import pytest
import torch

import plain_kefisun as plain
import trace_tools
from tiny_inference_server_b200.api import Engine, SamplingParams
from tiny_inference_server_b200.config import ConfigError, EngineConfig, KefisunConfig
from tiny_inference_server_b200.registry import build_model, config_from_dict, config_from_folder
from tiny_inference_server_b200.trace import TraceReplayer, make_runner

# ------------------------------------------------------------------------------------------------
# configurations: every size differs between them; K2 has sizes that are equal or 1 where K1's differ
# ------------------------------------------------------------------------------------------------


def _attn(heads, kv, dim, vdim, window, conv, v_mix=True, scale=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv, "scale": scale or dim ** -0.5,
         "v_mix": v_mix}
    if window is not None:
        m["mask"] = {"size": window}
    return m


def _delta(heads, kv, dim, vdim, conv, ranks):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv, "decay_rank": ranks[0],
            "gate_rank": ranks[1]}


def _ff(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


K1 = dict(architecture="Kefisun", vocab=131, width=64, canon={"taps": 3}, embedding={"scale": 3.0}, logit_scale=0.5,
          norm={"eps": 1e-5}, layers=[
              {"type": "attention", "mixer": _attn(4, 2, 16, 24, 9, 2), "mlp": _ff(80, 1.5)},
              {"type": "channel_delta", "mixer": _delta(4, 2, 16, 8, 4, (8, 16)), "mlp": None},
              {"type": "attention", "mixer": _attn(4, 2, 16, 24, 9, 2), "mlp": _ff(80, 1.5)},
              {"type": "attention", "mixer": _attn(2, 1, 8, 16, 21, 5, v_mix=False, scale=0.2), "mlp": None},
              {"type": "channel_delta", "mixer": _delta(2, 2, 24, 40, 2, (16, 8)), "mlp": _ff(48, 0.7)},
          ])
K2 = dict(architecture="Kefisun", vocab=67, width=32, canon={"taps": 2}, embedding={"scale": 1.0}, logit_scale=1.0,
          norm={"eps": 1e-6}, layers=[
              {"type": "channel_delta", "mixer": _delta(1, 1, 16, 16, 3, (8, 8)), "mlp": _ff(32, 2.0)},
              {"type": "attention", "mixer": _attn(1, 1, 16, 16, 16, 1), "mlp": None},
              {"type": "attention", "mixer": _attn(1, 1, 16, 16, 16, 1), "mlp": _ff(32, 2.0)},
          ])
K3 = dict(architecture="Kefisun", vocab=90, width=48, canon={"taps": 5}, embedding={"scale": 7.0}, logit_scale=2.0,
          norm={"eps": 1e-6}, layers=[
              {"type": "attention", "mixer": _attn(6, 3, 8, 8, None, 3), "mlp": _ff(40, 1.0)},
              {"type": "channel_delta", "mixer": _delta(3, 1, 12, 20, 4, (8, 24)), "mlp": _ff(40, 1.0)},
              {"type": "attention", "mixer": _attn(6, 3, 8, 8, 33, 3), "mlp": None},
          ])
# sizes that fit no vector, tile or alignment: every kernel's plain path, products with odd leading dimensions
K4 = dict(architecture="Kefisun", vocab=53, width=40, canon={"taps": 7}, embedding={"scale": 2.0}, logit_scale=1.5,
          norm={"eps": 1e-6}, layers=[
              {"type": "channel_delta", "mixer": _delta(2, 1, 6, 10, 6, (3, 5)), "mlp": _ff(27, 1.0)},
              {"type": "attention", "mixer": _attn(3, 1, 10, 6, 11, 6), "mlp": _ff(27, 1.0)},
              {"type": "attention", "mixer": _attn(3, 1, 10, 6, 11, 6), "mlp": None},
          ])
CONFIGS = {"K1": (K1, 16), "K2": (K2, 8), "K3": (K3, 12), "K4": (K4, 16)}
LENGTHS = {"K1": [1, 2, 3, 30, 75, 41, 9, 60], "K2": [1, 5, 40, 33, 17, 64], "K3": [2, 4, 50, 90, 23, 37],
           "K4": [3, 1, 45, 20, 70]}


def make_tensors(cfg, seed):
    """Weights of a size that makes every mechanism matter: projections of unit gain (queries and keys
    sharper), decays between nearly 0 and nearly 1, mixing weights away from 0 and 1; rounded to bfloat16
    so that both precisions and the plain implementation hold the same numbers."""
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, spec in build_model(cfg).expected_tensors().items():
        shape = tuple(spec.shape)
        leaf = name.split(".", 1)[1] if name.startswith("l") else name
        rnd = torch.randn(shape, generator=gen)
        uni = torch.rand(shape, generator=gen)
        if name == "embed":
            t = rnd * 0.5
        elif leaf in ("norm1", "norm2") or name == "final.norm":
            t = rnd * 0.2
        elif leaf.endswith(".conv") or leaf == "canon1":
            t = rnd * 0.5
        elif leaf in ("mix.q.norm", "mix.k.norm", "mix.norm"):
            t = 1.0 + rnd * 0.2
        elif leaf == "mix.r1":
            t = 0.2 + uni
        elif leaf == "mix.r2":
            t = 0.1 + 2.0 * uni
        elif leaf == "mix.vmix":
            t = 0.2 + 0.6 * uni
        elif leaf == "mix.A_log":
            t = -3.0 + 3.5 * uni
        elif leaf == "mix.dt_bias":
            t = -3.0 + 4.0 * uni
        elif leaf.endswith(".b") and len(shape) == 1:
            t = rnd * 0.3
        elif len(shape) == 2:
            gain = 2.0 if leaf in ("mix.q", "mix.k") else 1.0
            t = rnd * gain / math.sqrt(shape[1])
        else:
            raise AssertionError(f"no rule for {name} {shape}")
        out[name] = t.to(torch.bfloat16).contiguous()
    return out


def make_folder(raw, seed, folder):
    from safetensors.torch import save_file
    cfg = config_from_dict(json.loads(json.dumps(raw)))
    os.makedirs(folder, exist_ok=True)
    d = cfg.to_dict()
    for layer in d["layers"]:                      # the ranks are read back from the tensors' shapes
        layer["mixer"].pop("decay_rank", None)
        layer["mixer"].pop("gate_rank", None)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(d, f)
    save_file(make_tensors(cfg, seed), os.path.join(folder, "model.safetensors"))
    return folder


_cache = {}


def _setup(name, tmp_path_factory):
    if name not in _cache:
        raw, page = CONFIGS[name]
        folder = make_folder(raw, 11 + len(name) + ord(name[-1]), str(tmp_path_factory.mktemp(f"kefisun{name}")))
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


def _steps(mode, seqs, max_live=4):
    if mode == "whole":
        return trace_tools.trace_whole(seqs)
    if mode == "tail":
        return trace_tools.trace_tail(seqs, tail=32)
    if mode == "chunks":
        return trace_tools.trace_chunks(seqs)
    return trace_tools.trace_mixed(seqs, max_live=max_live)


def _replay_and_compare(raw, page, folder, seqs, ref, steps, out_dir, dtype, device, tol, max_live=4, poison=False,
                        shuffle=False):
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
    worst = 0.0
    for rid, toks in seqs.items():
        for p in range(len(toks)):
            e = rel_err(got[rid][p], ref[rid][p])
            assert e < tol, f"logits of {rid} at position {p}: relative error {e} (first wrong place)"
            worst = max(worst, e)
    return runner, worst


# ------------------------------------------------------------------------------------------------
# configuration and weights (CPU)
# ------------------------------------------------------------------------------------------------

def test_config_round_trip_and_ranks_from_shapes(tmp_path):
    folder = make_folder(K1, 1, str(tmp_path / "m"))
    cfg = config_from_folder(folder)
    assert isinstance(cfg, KefisunConfig)
    assert cfg.layers[1]["mixer"]["decay_rank"] == 8 and cfg.layers[1]["mixer"]["gate_rank"] == 16
    assert cfg.layers[4]["mixer"]["decay_rank"] == 16 and cfg.layers[4]["mixer"]["gate_rank"] == 8
    again = config_from_dict(cfg.to_dict())
    assert again.to_dict() == cfg.to_dict()
    model = build_model(cfg)
    names = set(model.expected_tensors())
    assert {"embed", "final.norm", "l0.canon1", "l0.mix.q.conv", "l0.mix.vmix", "l1.mix.A_log", "l0.mlp.down.b"} <= names
    assert "l1.norm2" not in names and "l3.mix.vmix" not in names


def test_config_errors_name_the_problem():
    bad = json.loads(json.dumps(K2))
    bad["layers"][0]["type"] = "conv_only"
    with pytest.raises(ConfigError, match="layers\\[0\\].type"):
        config_from_dict(bad)
    bad = json.loads(json.dumps(K2))
    bad["layers"][1]["mixer"]["heads"] = 3
    bad["layers"][1]["mixer"]["kv_heads"] = 2
    with pytest.raises(ConfigError, match="not a multiple"):
        config_from_dict(bad)
    bad = json.loads(json.dumps(K2))
    bad["depth"] = 3
    with pytest.raises(ConfigError, match="unknown keys: depth"):
        config_from_dict(bad)


# ------------------------------------------------------------------------------------------------
# the engine's plumbing on the CPU
# ------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("name", ["K1", "K2", "K3", "K4"])
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
    raw, page, folder, seqs, ref, c, W = _setup("K2", tmp_path_factory)
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
OP_TOL = {"float32": 2e-5, "bfloat16": 2e-2}


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
@pytest.mark.parametrize("taps,silu,residual", [(4, False, True), (2, True, False), (1, False, False), (7, True, False)])
def test_causal_conv_in_portions(dtype, taps, silu, residual):
    """Two sequences fed in portions of 1..9 rows, side by side in one step and in slots 2 and 0: what the state
    carries over equals the convolution of the whole sequence."""
    from tiny_inference_server_b200.kernels import ops
    torch.manual_seed(taps)
    C, L = 37, 40
    w = torch.randn(C, taps)
    xs = [torch.randn(L, C).to(DT[dtype]) for _ in range(2)]
    ref = []
    for x in xs:
        y = plain.causal_conv(x.double(), w.double())
        if residual:
            y = y + x.double()
        ref.append(plain.silu(y) if silu else y)
    state = torch.full((3, (taps - 1) * C + 5), 0.0, device="cuda")
    state[1] = 7.0                                   # a slot that nobody uses keeps what it holds
    got = [torch.zeros(L, C, dtype=DT[dtype], device="cuda") for _ in range(2)]
    fed = [0, 0]
    sizes = [(3, 1), (1, 2), (2, 9), (9, 1), (1, 1), (5, 3), (2, 2), (17, 21)]
    for a, b in sizes:
        cuts = [min(a, L - fed[0]), min(b, L - fed[1])]
        x = torch.cat([xs[0][fed[0]:fed[0] + cuts[0]], xs[1][fed[1]:fed[1] + cuts[1]]]).cuda()
        out = torch.empty_like(x)
        row_slot, row_last = _rows(cuts, [2, 0])
        ops.causal_conv(x, w.t().contiguous().cuda(), state, out, row_slot, row_last, residual=residual, silu=silu)
        got[0][fed[0]:fed[0] + cuts[0]] = out[:cuts[0]]
        got[1][fed[1]:fed[1] + cuts[1]] = out[cuts[0]:]
        fed = [fed[0] + cuts[0], fed[1] + cuts[1]]
    assert fed == [L, L]
    for g, r in zip(got, ref):
        _close(g, r, OP_TOL[dtype], "convolution")
    assert float(state[1].min()) == 7.0


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_norms_embedding_gating(dtype):
    from tiny_inference_server_b200.kernels import ops
    torch.manual_seed(0)
    n, d, F = 5, 52, 19
    res = torch.randn(n, d, device="cuda") * 3
    delta = torch.randn(n, d, device="cuda").to(DT[dtype])
    w = torch.randn(d, device="cuda") * 0.3
    out = torch.empty(n, d, dtype=DT[dtype], device="cuda")
    total = res.double().cpu() + delta.double().cpu()
    ops.add_rmsnorm(res, delta, (1.0 + w).contiguous(), 1e-3, out, kind="mean_eps")
    _close(out, plain.norm_one_plus(total, w.double().cpu(), 1e-3), OP_TOL[dtype], "norm")
    _close(res, total, 1e-6, "stream")
    table = torch.randn(11, d).to(DT[dtype]).cuda()
    tok = torch.tensor([3, 0, 10], dtype=torch.int32, device="cuda")
    emb = torch.empty(3, d, device="cuda")
    ops.embed_rows(table, tok, emb, 2.5)
    _close(emb, table.double().cpu()[[3, 0, 10]] * 2.5, 1e-6, "embedding")
    gu = (torch.randn(n, 2 * F, device="cuda") * 2).to(DT[dtype])
    bg, bu = torch.randn(F, device="cuda"), torch.randn(F, device="cuda")
    y = torch.empty(n, 24, dtype=DT[dtype], device="cuda")
    ops.glu_clamped(gu, bg, bu, 1.25, 1.702, 1.0, y, F)
    g = (gu[:, :F].double().cpu() + bg.double().cpu()).clamp(max=1.25)
    u = (gu[:, F:].double().cpu() + bu.double().cpu()).clamp(min=-1.25, max=1.25)
    _close(y[:, :F], g * torch.sigmoid(1.702 * g) * (u + 1), OP_TOL[dtype], "gating")
    assert y[:, F].float().eq(1).all() and y[:, F + 1:].float().eq(0).all()
    x = torch.randn(7, 9, device="cuda")
    want = x.double().cpu() * 0.3
    _close(ops.scale_f32(x, 0.3), want, 1e-6, "scaling")


class _Step:
    """What an attention kernel asks of a step, for one request's portion outside the engine."""
    decode_only = False

    def __init__(self, positions, row_slot):
        self.positions, self.row_slot = positions, row_slot

    def plan(self, planner):
        return planner.infer(self.positions, self.row_slot)


def _paged(n_pages, kv, page, k_dim, v_dim, dtype):
    kp = torch.full((n_pages, kv, page, k_dim), 1e4, dtype=DT[dtype], device="cuda")
    vp = torch.full((n_pages, kv, page, v_dim), 1e4, dtype=DT[dtype], device="cuda")
    return kp, vp


def _plain_attention(q, k, v, gate, H, G, scale, r1, r2, window):
    """Rows of one sequence: q (L, H*kd), k (L, G*kd), v (L, G*vd) float64."""
    L = q.shape[0]
    kd, vd = q.shape[1] // H, v.shape[1] // G
    qh = q.view(L, H, kd).transpose(0, 1)
    kh = k.view(L, G, kd).transpose(0, 1).repeat_interleave(H // G, dim=0)
    vh = v.view(L, G, vd).transpose(0, 1).repeat_interleave(H // G, dim=0)
    s = qh @ kh.transpose(1, 2) * scale - plain.distance_bias(r1, r2, L)
    s = s.masked_fill(~plain.window_mask(L, window), float("-inf"))
    o = (torch.softmax(s, -1) @ vh).transpose(0, 1).reshape(L, H * vd)
    return o * torch.sigmoid(gate)


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,kd,vd,window,page", [(4, 2, 16, 24, 9, 4), (6, 2, 48, 32, 40, 16), (2, 2, 8, 160, None, 8),
                                                   (3, 1, 20, 12, 130, 16), (4, 1, 32, 16, 70, 8), (2, 2, 128, 64, 100, 16),
                                                   (2, 1, 16, 16, None, 16)])
def test_window_attention_with_planted_keys(dtype, H, G, kd, vd, window, page):
    """norm + mix + store, then attention, in portions and single rows over scattered pages.  One key a few
    positions back and the keys at distance window - 1 and window from chosen rows are made to stand out (a
    large key along the row's query): the first two are seen, the third is not, in a portion and in a row
    decoded alone, and at the first and last place of a page."""
    from tiny_inference_server_b200.kernels import ops
    torch.manual_seed(H * 100 + kd)
    L = 3 * (window or 50) + 7
    nq, nk, nv = H * kd, G * kd, G * vd
    q = torch.randn(L, nq)
    k = torch.randn(L, nk)
    v = torch.randn(L, nv)
    marks = []
    if window:
        for row in (window + 3, 2 * window + page - (2 * window) % page, L - 1):      # the last: a row fed alone
            if row >= L:
                continue
            for dist in (window - 1, window):
                j = row - dist
                if j < 0:
                    continue
                k[j, :kd] = q[row, :kd] * 3.0          # kv head 0 <- the row's query head 0
                v[j] += 5.0
                marks.append((row, j))
    q, k, v = q.to(DT[dtype]), k.to(DT[dtype]), v.to(DT[dtype])
    v_other = torch.randn(L, nv).to(DT[dtype])
    gate = torch.randn(L, H * vd).to(DT[dtype])
    wq, wk = 1 + 0.2 * torch.randn(nq), 1 + 0.2 * torch.randn(nk)
    lam = torch.tensor([0.3])
    r1, r2 = 0.2 + torch.rand(H), 0.1 + torch.rand(H)
    eps, scale = 1e-5, 0.5 * kd ** -0.5
    qn = plain.rms(q.double(), eps) * wq.double()
    kn = plain.rms(k.double(), eps) * wk.double()
    vm = 0.7 * v.double() + 0.3 * v_other.double()
    if dtype == "bfloat16":      # what the cache holds is rounded
        qn, kn, vm = (t.to(torch.bfloat16).double() for t in (qn, kn, vm))
    ref = _plain_attention(qn, kn, vm, gate.double(), H, G, scale, r1.double(), r2.double(), window)
    n_pages = (L + page - 1) // page + 3
    kp, vp = _paged(n_pages, G, page, kd, vd, dtype)
    perm = torch.randperm(n_pages)[: (L + page - 1) // page].to(torch.int32)
    table = torch.full((3, len(perm) + 2), -1, dtype=torch.int32)
    table[1, :len(perm)] = perm
    table = table.cuda()
    fault = torch.zeros(4, dtype=torch.int32, device="cuda")
    got = torch.zeros(L, H * vd, dtype=DT[dtype], device="cuda")
    before = ops.calls["window_attention_mma"]
    fed = 0
    cuts = [5, 2, 1, 1, 30, 2, 64, 100]
    i = 0
    while fed < L:
        n = min(cuts[i % len(cuts)], L - fed) if fed < L - 1 - 3 else 1
        n = min(n, max(1, L - 4 - fed)) if fed < L - 4 else 1
        i += 1
        rows = slice(fed, fed + n)
        qkv = torch.cat([q[rows], k[rows], v[rows]], dim=1).cuda().contiguous()
        pos = torch.arange(fed, fed + n, dtype=torch.int32, device="cuda")
        slot = torch.full((n,), 1, dtype=torch.int32, device="cuda")
        ops.norm_mix_store(qkv, nq, nk, nv, wq.cuda(), wk.cuda(), eps, v_other[rows].cuda(), lam.cuda(), kp, vp, table, pos,
                           slot, page, fault)
        out = torch.empty(n, H * vd, dtype=DT[dtype], device="cuda")
        # portions as a step of the engine (in bfloat16, with widths that are multiples of 16: the tensor-core kernel)
        ops.window_attention(qkv[:, :nq], gate[rows].cuda(), out, kp, vp, table, pos, slot, H, page, window, scale,
                             r1.cuda(), r2.cuda(), fault, step=_Step(pos, slot) if n != 2 else None)
        got[rows] = out
        fed += n
    assert int(fault[0]) == 0
    if dtype == "bfloat16" and kd % 16 == 0 and vd % 16 == 0:
        assert ops.calls["window_attention_mma"] > before
    _close(got, ref, 4e-2 if dtype == "bfloat16" else 1e-4, "attention")
    # the planted keys matter: the plain result with a window one longer or shorter differs at those rows
    for w_off in (-1, 1):
        if window:
            other = _plain_attention(qn, kn, vm, gate.double(), H, G, scale, r1.double(), r2.double(), window + w_off)
            for row in {m[0] for m in marks}:
                assert float((other[row] - ref[row]).abs().max()) > 0.05


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,kd,vd", [(4, 2, 16, 8), (2, 2, 24, 40), (3, 1, 32, 64), (1, 1, 128, 96), (2, 1, 12, 20)])
def test_delta_rule_in_portions_and_far_memory(dtype, H, G, kd, vd):
    """The recurrence over portions of 1..70 rows equals the token-by-token rule on the whole sequence.  Head 0
    hardly decays and is written strongly at position 1 only: its read-out 250 tokens later still is that value."""
    from tiny_inference_server_b200.kernels import ops
    torch.manual_seed(kd + vd)
    L = 260
    nq, nv, na = G * kd, H * vd, H * kd
    qkv = torch.randn(L, 2 * nq + nv)
    beta = torch.randn(L, H)
    a = torch.randn(L, na)
    a_log = -1.0 + torch.rand(H)
    dt_bias = -1.0 + torch.rand(na)
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
    # plain rule
    q = qkv[:, :nq].double().view(L, G, kd)
    k = qkv[:, nq:2 * nq].double().view(L, G, kd)
    v = qkv[:, 2 * nq:].double().view(L, H, vd)
    q = (q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * kd ** -0.5).repeat_interleave(H // G, dim=1)
    k = (k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)).repeat_interleave(H // G, dim=1)
    decay = torch.exp(-torch.exp(a_log.double())[None, :, None] *
                      torch.nn.functional.softplus(a.double().view(L, H, kd) + dt_bias.double().view(H, kd)))
    b = torch.sigmoid(beta.double())
    S = torch.zeros(H, kd, vd, dtype=torch.float64)
    o = torch.zeros(L, H, vd, dtype=torch.float64)
    for t in range(L):
        S = decay[t][:, :, None] * S
        u = b[t][:, None] * (v[t] - torch.einsum("hdv,hd->hv", S, k[t]))
        S = S + k[t][:, :, None] * u[:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    raw_far = o[L - 3, 0].clone()
    ref = (plain.rms(o, eps) * norm_w.double() * torch.sigmoid(gate.double().view(L, H, vd))).reshape(L, nv)
    # the far value really is the one written at position 1
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
                       requests=1 if i % 2 else None)     # few requests: the kernel with narrow column slices
        got[rows] = out
        fed += n
    _close(got, ref, 3e-2 if dtype == "bfloat16" else 1e-4, "delta rule")
    _close(state[2, :H * kd * vd], S.reshape(-1), 1e-4, "state")
    assert float(state[0].abs().max()) == 0 and float(state[2, H * kd * vd:].abs().max()) == 0


# ------------------------------------------------------------------------------------------------
# GPU: the whole model through the engine
# ------------------------------------------------------------------------------------------------

@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["K1", "K2", "K3", "K4"])
@pytest.mark.parametrize("mode", ["whole", "tail", "chunks", "mixed"])
def test_replay_gpu(name, mode, dtype, tmp_path, tmp_path_factory):
    raw, page, folder, seqs, ref, _, _ = _setup(name, tmp_path_factory)
    steps = _steps(mode, seqs, max_live=3)
    runner, _ = _replay_and_compare(raw, page, folder, seqs, ref, steps, str(tmp_path / "out"), dtype, "cuda:0", TOL[dtype],
                                    max_live=3, poison=(mode == "mixed"), shuffle=(mode == "mixed"))
    if mode == "mixed" and name == "K1":          # its requests are long enough for the pool to turn over
        pool = runner.cache.groups[0].pool
        assert pool.allocations > pool.num_pages, "the trace does not use pages again"


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_two_slots_used_again_and_again(dtype, tmp_path, tmp_path_factory):
    """Eight requests through two state slots: a state that is not cleared, or a slot's convolution history that
    leaks into the next request, shows in the first tokens of the later requests."""
    raw, page, folder, seqs, ref, _, _ = _setup("K1", tmp_path_factory)
    steps = trace_tools.trace_mixed(seqs, max_live=2, prefill_sizes=(2, 7, 3, 2), skip_every=4)
    _replay_and_compare(raw, page, folder, seqs, ref, steps, str(tmp_path / "out"), dtype, "cuda:0", TOL[dtype], max_live=2,
                        poison=True)


@gpu
def test_long_decoding_float32(tmp_path, tmp_path_factory):
    """A short prompt, then 300 tokens one by one: the windows (9 and 21 keys) pass over decoded tokens many
    times, pages behind them are given back and used again (the pool holds 64 tokens), decode steps are replayed
    from a graph."""
    raw, page, folder, _, _, c, W = _setup("K1", tmp_path_factory)
    g = torch.Generator().manual_seed(9)
    toks = torch.randint(0, raw["vocab"], (305,), generator=g).tolist()
    ref = {"a": plain.plain_forward(c, W, toks).numpy()}
    steps = trace_tools.trace_tail({"a": toks}, tail=300)
    runner = make_runner(folder, "float32", 64, page_size=page, max_live=1, debug_poison=True)
    out_dir = str(tmp_path / "out")
    TraceReplayer(runner, out_dir).run(json.dumps(s) for s in steps)
    assert runner.cache.drained()
    assert runner.graphs is not None and runner.graphs.replays > 250
    got = trace_tools.gather(steps, out_dir, raw["vocab"])
    for p in range(len(toks)):
        assert rel_err(got["a"][p], ref["a"][p]) < TOL["float32"], f"position {p}"


@gpu
def test_generate_through_the_scheduler(tmp_path, tmp_path_factory):
    raw, page, folder, seqs, _, c, W = _setup("K3", tmp_path_factory)
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
    and fed again from their first token (their recurrent state and convolution histories start from zero again)."""
    from test_cli import _cli, _ids
    raw, page, folder, seqs, _, c, W = _setup("K3", tmp_path_factory)
    new = 8
    prompts = [seqs["r0"], seqs["r4"], seqs["r1"]]
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
