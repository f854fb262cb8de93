"""Kusolorn through the engine against the plain implementation (``plain_kusolorn``), mechanism by mechanism and as a
whole: every way of cutting the work, pages and state slots that are used again, keys just inside and just outside the
window and the kept first tokens, sizes that are odd, equal to one or absent, and greedy generation through the entry
point and the scheduler.
"""
from __future__ import annotations

import json
import math
import os

import numpy as np
import pytest
import torch

import plain_kusolorn as plain
import traces
from conftest import note_error, random_tokens

pytestmark = pytest.mark.gpu


def _attention(heads, kv_heads, dim, vdim, scale, window=None, keep=0, rot=None, softcap=None, v_mix=False, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "softcap": softcap, "v_mix": v_mix}
    if window:
        m["mask"] = {"size": window, "keep_first": keep}
    if rot:
        m["rot"] = rot
    return {"type": "attention", "mixer": m, "mlp": mlp}


def _moe(experts, top, ff, limit):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": limit}}


def _config(vocab, width, layers, side=None, eps=1e-6):
    cfg = {"architecture": "Kusolorn", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if side:
        cfg["token_side"] = {"dim": side}
    return cfg


SCALED = {"base": 500.0, "dims": 8, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}}
# odd sizes everywhere; every mixer; a window of 9 that keeps 2 tokens and one of 17 that keeps none; a layer without
# feed-forward; one key/value head; the second value-mixing layer has other key sizes than the first
ODD = _config(97, 72, [
    _attention(3, 1, 24, 20, 0.45, window=9, keep=2, rot=SCALED, softcap=30.0, v_mix=True, mlp={"kind": "dense", "ff": 100}),
    {"type": "delta", "mixer": {"heads": 4, "kv_heads": 2, "dim": 12, "vdim": 20, "conv": 4}, "mlp": _moe(5, 2, 36, 0.7)},
    {"type": "mlstm", "mixer": {"heads": 3, "dim": 20, "vdim": 12, "gate_cap": 8.0}, "mlp": None},
    _attention(2, 1, 16, 20, 0.6, window=17, keep=0, rot={"base": 100.0, "dims": 16}, v_mix=True, mlp=_moe(3, 3, 24, 2.0)),
], side=10, eps=1e-5)
# the recurrent mixers first, attention without a window and without rotation, no per-layer token input, one tap (no
# convolution state), as many key heads as value heads, one expert per token, pages of 32
LATE = _config(300, 128, [
    {"type": "mlstm", "mixer": {"heads": 1, "dim": 40, "vdim": 72, "gate_cap": 15.0}, "mlp": _moe(4, 1, 64, 1.0)},
    {"type": "delta", "mixer": {"heads": 2, "kv_heads": 2, "dim": 32, "vdim": 32, "conv": 1}, "mlp": {"kind": "dense", "ff": 256}},
    _attention(4, 4, 32, 16, 0.3, mlp={"kind": "dense", "ff": 96}),
    _attention(4, 2, 32, 48, 0.3, window=33, keep=40, rot={"base": 10000.0, "dims": 32}, softcap=8.0, v_mix=True, mlp=None),
])
# sizes in multiples of 64, for the tensor-core paths in bfloat16 (grouped experts, tcgen05 projections)
WIDE = _config(768, 384, [
    _attention(12, 4, 64, 64, 0.2, window=48, keep=5, rot={"base": 5e5, "dims": 16, "scaling": {"factor": 4.0, "low": 1.0, "high": 8.0, "original": 256}},
               softcap=40.0, v_mix=True, mlp=_moe(6, 2, 128, 1.0)),
    {"type": "delta", "mixer": {"heads": 4, "kv_heads": 2, "dim": 64, "vdim": 64, "conv": 4}, "mlp": {"kind": "dense", "ff": 768}},
    _attention(4, 4, 128, 64, 0.12, window=64, keep=16, rot={"base": 1e4, "dims": 64}, v_mix=True, mlp=_moe(8, 3, 64, 3.0)),
    {"type": "mlstm", "mixer": {"heads": 3, "dim": 64, "vdim": 128, "gate_cap": 9.0}, "mlp": {"kind": "dense", "ff": 384}},
], side=16)
MODELS = {"odd": (ODD, 16, 21), "late": (LATE, 32, 22), "wide": (WIDE, 16, 23)}

# Largest error of a row of logits (see _row_error).  float32: only the order of sums differs.  bfloat16: the engine
# rounds where it stores (normed rows, projections, cached keys and values, mixer outputs, activations).
TOLERANCE = {"float32": 4e-5, "bfloat16": 8e-2}


def _write(folder, cfg, tensors, dtype):
    from cuinfer_b200.weights.safetensors_io import write_safetensors

    os.makedirs(folder, exist_ok=True)
    store = {k: v.to(torch.bfloat16 if dtype == "bfloat16" else torch.float32) for k, v in tensors.items()}
    write_safetensors(os.path.join(folder, "model.safetensors"), store)
    with open(os.path.join(folder, "config.json"), "w") as fh:
        json.dump(cfg, fh)
    return folder


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    """{name: (config, {dtype: folder}, tensors in float64, page size)}; the values are bfloat16 numbers, so that both
    engines and the plain implementation read the same weights."""
    out = {}
    for name, (cfg, block, seed) in MODELS.items():
        tensors = plain.random_model(cfg, seed)
        dirs = {d: _write(str(tmp_path_factory.mktemp(f"kusolorn_{name}_{d}")), cfg, tensors, d) for d in TOLERANCE}
        out[name] = (cfg, dirs, {k: v.double() for k, v in tensors.items()}, block)
    return out


def _row_error(row, ref):
    """Root mean square of the difference over the vocabulary, the common offset taken off (it changes no probability),
    as a fraction of the root mean square of the plain logits about their mean."""
    d = row.astype(np.float64) - ref
    return float(np.sqrt(((d - d.mean()) ** 2).mean()) / np.sqrt(((ref - ref.mean()) ** 2).mean()))


def _requests(cfg, lengths, seed):
    return {f"r{i}": random_tokens(cfg["vocab"], n, seed * 100 + i) for i, n in enumerate(lengths)}


# Between two ways of cutting the same request the engine may differ only by which kernel a step's size selects
# (float32 has one kernel per operation, so there the logits agree to the last bits; in bfloat16 the kernels of a step of
# few rows and of many round at different places, which moves a row as much as rounding moves it against the plain one).
CUT_TOLERANCE = {"float32": 2e-6, "bfloat16": 8e-2}
_WHOLE = {}


def _whole_rows(folders, name, dtype, rid, toks, tmp_path):
    """The engine's own logits of a request fed whole and alone."""
    key = (name, dtype, tuple(toks))
    if key not in _WHOLE:
        cfg, dirs, _tensors, block = folders[name]
        steps = traces.whole({rid: toks})
        out = str(tmp_path / f"whole_{name}_{dtype}_{rid}")
        traces.replay_in_process(dirs[dtype], dtype, steps, out, traces.live_token_peak(steps), block)
        _WHOLE[key] = traces.collect(steps, out, cfg["vocab"])[rid]
    return _WHOLE[key]


def _check(folders, name, dtype, steps, requests, tmp_path, max_tokens=None, **kw):
    """Every row against the plain implementation, and against the engine's own logits of the request fed whole.  A few
    positions are ill-conditioned in the design itself (a recurrent mixer's first read-outs are a vector times ONE dot
    product, whose sign and size then pass through the head norm): up to one position in fifty of a request may be off
    by up to four times the bound against the plain implementation (and, in bfloat16, against the engine's other kernels);
    in float32 the engine agrees with itself at every position, however the work is cut."""
    cfg, dirs, tensors, block = folders[name]
    out = str(tmp_path / f"out_{name}_{dtype}")
    runner = traces.replay_in_process(dirs[dtype], dtype, steps, out, max_tokens or traces.live_token_peak(steps), block, **kw)
    got = traces.collect(steps, out, cfg["vocab"])
    worst = 0.0
    for rid, toks in requests.items():
        assert plain.router_margin(cfg, tensors, list(toks)) > 0.03, "the test's routers must not rest on a close call"
        ref = plain.forward(cfg, tensors, list(toks)).numpy()
        assert got.get(rid), f"no logits came back for request {rid}"
        assert sorted(got[rid]) == list(range(len(toks)))
        whole = _whole_rows(folders, name, dtype, rid, list(toks), tmp_path)
        over = []
        for pos, row in sorted(got[rid].items()):
            assert np.isfinite(row).all(), f"request {rid} position {pos}: logits are not finite"
            cut = _row_error(row, whole[pos].astype(np.float64))
            sharp = dtype == "float32"          # in bfloat16 an ill-conditioned position moves with the kernels a step's size selects
            assert cut <= CUT_TOLERANCE[dtype] * (1 if sharp else 4), f"{name}/{dtype}: request {rid}: position {pos} of {len(toks)} depends on how the work was cut ({cut:.3e})"
            err = _row_error(row, ref[pos])
            assert err <= 4 * TOLERANCE[dtype], f"{name}/{dtype}: request {rid}: first wrong position {pos} of {len(toks)} (error {err:.3e})"
            if err > TOLERANCE[dtype] or cut > CUT_TOLERANCE[dtype]:
                over.append(pos)
            else:
                worst = max(worst, err)
        assert len(over) <= max(1, len(toks) // 50), f"{name}/{dtype}: request {rid}: positions {over} of {len(toks)} are over the bound"
    note_error(dtype, f"model {name}", worst, family="Kusolorn")
    return runner


NAMES, DTYPES = list(MODELS), list(TOLERANCE)


# ---- the whole model under every way of cutting the work ------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_prompts(folders, name, dtype, tmp_path):
    requests = _requests(folders[name][0], [1, 2, 17, 33, 150], seed=1)
    _check(folders, name, dtype, traces.whole(requests), requests, tmp_path)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_prefill_then_token_by_token(folders, name, dtype, tmp_path):
    """The decoded tail is longer than every window, so windows pass over decoded tokens and pages are given back."""
    requests = _requests(folders[name][0], [40, 131], seed=2)
    _check(folders, name, dtype, traces.tail_decode(requests, 70), requests, tmp_path)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_portions_down_to_two_tokens(folders, name, dtype, tmp_path):
    requests = _requests(folders[name][0], [64, 131, 90], seed=3)
    _check(folders, name, dtype, traces.portions(requests), requests, tmp_path)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_mixed_batches_reuse_pages_and_slots(folders, name, dtype, tmp_path):
    requests = _requests(folders[name][0], [70, 33, 120, 58, 90, 45, 101], seed=4)
    steps = traces.mixed(requests, max_live=4)
    peak = traces.live_token_peak(steps)
    assert peak < sum((len(t) + 63) // 64 * 64 for t in requests.values()), "pages must be used again"
    runner = _check(folders, name, dtype, steps, requests, tmp_path, max_tokens=peak, max_live=4)
    assert runner.num_pages * runner.page_size == peak and runner.manager.slots.num_slots == 4


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_from_the_first_token(folders, dtype, tmp_path):
    requests = _requests(folders["odd"][0], [260], seed=5)
    _check(folders, "odd", dtype, traces.tail_decode(requests, 259), requests, tmp_path)


@pytest.mark.parametrize("dtype", DTYPES)
def test_steps_through_cuda_graphs(folders, dtype, tmp_path):
    """The same logits when decode steps and repeated step shapes are replayed from graphs, as generation runs them:
    padding rows and the padding request own no state slot and no page."""
    requests = _requests(folders["wide"][0], [70, 40, 90, 33], seed=6)
    steps = traces.mixed(requests, max_live=3, sizes=(32, 40, 35))
    _check(folders, "wide", dtype, steps, requests, tmp_path, cuda_graph=True, passes=2, max_live=4)


def test_greedy_generation_through_the_entry_point(folders):
    from cuinfer_b200 import LLM, SamplingParams

    for name in ("odd", "late"):
        cfg, dirs, tensors, block = folders[name]
        prompts = [random_tokens(cfg["vocab"], n, 70 + n) for n in (3, 19, 8)]
        llm = LLM(dirs["float32"], dtype="float32", block_size=block, num_blocks=24, max_num_seqs=3, max_num_scheduled_tokens=16)
        outs = llm.generate(prompts, SamplingParams(max_tokens=12, temperature=0.0, ignore_eos=True))
        for prompt, out in zip(prompts, outs):
            assert out.token_ids == plain.greedy(cfg, tensors, prompt, 12), f"{name}: prompt of {len(prompt)} tokens"


def test_command_line(folders):
    import subprocess
    import sys

    from conftest import ROOT

    cfg, dirs, tensors, block = folders["late"]
    prompt = random_tokens(cfg["vocab"], 9, 95)
    proc = subprocess.run([sys.executable, "-m", "cuinfer_b200", "generate", "--model", dirs["float32"], "--dtype", "float32",
                           "--prompt-ids", ",".join(map(str, prompt)), "--max-tokens", "5", "--temperature", "0", "--ignore-eos",
                           "--num-blocks", "16", "--max-num-seqs", "4", "--block-size", str(block)],
                          capture_output=True, text=True, cwd=ROOT, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    line = [json.loads(l) for l in proc.stdout.splitlines() if l.startswith("{")][0]
    assert line["token_ids"] == plain.greedy(cfg, tensors, prompt, 5)


# ---- mechanisms alone -------------------------------------------------------------------------------------------------
def _dev(t, dtype):
    return t.to(device="cuda", dtype=dtype).contiguous()


def _close(got, want, dtype, what, tol=None):
    tol = tol or (2e-5 if dtype == torch.float32 else 2e-2)
    err = float((got.double().cpu() - want).abs().max() / want.abs().max().clamp_min(1e-9))
    assert err <= tol, f"{what} in {dtype}: error {err:.3e} of the largest value"


def _ints(values):
    return torch.tensor(values, dtype=torch.int32, device="cuda")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width", [8, 37, 72, 1000, 4100])
def test_rms_norm_on_both_sides_in_one_pass(dtype, width):
    from cuinfer_b200 import kernels

    g = torch.Generator().manual_seed(width)
    rows = 5
    res = torch.randn(rows, width, generator=g, dtype=torch.float64) * 3
    y = (torch.randn(rows, width, generator=g) * 7 + 2).to(dtype).double()
    gains = [(1 + 0.2 * torch.randn(width, generator=g)).bfloat16().double() for _ in range(2)]
    x = res + plain.rms_norm(y, gains[0], 1e-5)
    d_res = _dev(res, torch.float32)
    out, raw = torch.empty(rows, width, dtype=dtype, device="cuda"), torch.empty(rows, width, dtype=dtype, device="cuda")
    v = [_dev(t, torch.bfloat16) for t in gains]
    kernels.rms_stream(d_res, _dev(y, dtype), (v[0], 1e-5), (v[1], 1e-3), out, raw=raw)
    _close(d_res, x, torch.float32, "residual after the output norm and the sum")
    _close(out, plain.rms_norm(x, gains[1], 1e-3), dtype, "input norm")
    _close(raw, x, dtype, "the stream itself")
    d_res2 = _dev(res, torch.float32)
    kernels.rms_stream(d_res2, _dev(y, dtype), None, None, None)
    _close(d_res2, res + y, torch.float32, "plain delta")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gelu_with_and_without_the_token_table(dtype):
    from cuinfer_b200 import kernels

    g = torch.Generator().manual_seed(4)
    x = (torch.randn(7, 13, generator=g) * 3).to(dtype).double()
    table = torch.randn(11, 40, generator=g).to(dtype)
    ids = [3, 0, 10, 10, 7, 1, 2]
    out = torch.empty(7, 13, dtype=dtype, device="cuda")
    kernels.gelu_tanh(_dev(x, dtype), out)
    _close(out, plain.gelu_tanh(x), dtype, "gelu")
    kernels.gelu_tanh(_dev(x, dtype), out, table.cuda()[:, 13:26], _ints(ids))
    _close(out, plain.gelu_tanh(x) * table.double()[ids, 13:26], dtype, "gelu times the token's columns")


@pytest.mark.parametrize("experts,top", [(5, 2), (3, 3), (16, 4), (70, 1), (130, 9)])
def test_router_choice_and_weights(experts, top):
    from cuinfer_b200 import kernels

    g = torch.Generator().manual_seed(experts)
    z = torch.randn(33, experts, generator=g) * 3
    z[5, :] = 1.25                                   # a tie everywhere: the lowest indices win
    choice = torch.empty(33, top, dtype=torch.int32, device="cuda")
    weight = torch.empty(33, top, dtype=torch.float32, device="cuda")
    kernels.router_topk(z.cuda(), top, choice, weight)
    vals, idx = torch.topk(z.double(), top, dim=-1)
    assert choice.cpu()[5].tolist() == list(range(top))
    rows = [r for r in range(33) if r != 5]
    assert torch.equal(choice.cpu()[rows].long(), idx[rows])
    _close(weight[rows], torch.softmax(vals, -1)[rows], torch.float32, "weights over the chosen logits")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,width,ff,experts,top", [(5, 40, 24, 4, 2), (300, 64, 96, 5, 3), (9, 72, 20, 3, 1)])
def test_routed_experts_with_the_clamped_gate(dtype, rows, width, ff, experts, top):
    """Few rows (a product per token and choice) and many (grouped by expert on the tensor cores); an expert that gets
    no row at all; the limit reached on both sides."""
    from cuinfer_b200 import kernels

    g = torch.Generator().manual_seed(rows)
    h = (torch.randn(rows, width, generator=g) * 2).to(dtype).double()
    gate_up = (torch.randn(experts, 2 * ff, width, generator=g) / math.sqrt(width)).bfloat16().double()
    down = (torch.randn(experts, width, ff, generator=g) / math.sqrt(ff)).bfloat16().double()
    choice = torch.stack([torch.randperm(experts - 1, generator=g)[:top] for _ in range(rows)]).to(torch.int32)   # the last expert: no row
    weight = torch.softmax(torch.randn(rows, top, generator=g), -1)
    limit = 0.8
    want = torch.zeros(rows, width, dtype=torch.float64)
    for t in range(rows):
        for c in range(top):
            e = int(choice[t, c])
            want[t] += weight[t, c].double() * plain.expert_ff(h[t:t + 1], gate_up[e, :ff], gate_up[e, ff:], down[e], limit)[0]
    out = torch.empty(rows, width, dtype=dtype, device="cuda")
    kernels.moe_table_feed_forward(_dev(h, dtype), None, choice.cuda(), _dev(gate_up, dtype), _dev(down, dtype), None, out,
                                   weights=weight.cuda(), clamp_limit=limit)
    _close(out, want, dtype, "weighted sum of the chosen experts", tol=None if dtype == torch.float32 else 3e-2)


def _attention_case(dtype, H, G, d, dv, lengths, new, page, seed, window, keep, cap, sharpen=None, tensor_cores=False, splits=1):
    """Requests of ``lengths`` tokens whose last ``new`` are this step's queries, over a cache of random keys and values
    on shuffled pages; kernel output and the plain result from the same cached rows.  ``sharpen[t] = j`` makes query t's
    score with key j of its request stand out."""
    from cuinfer_b200 import kernels

    g = torch.Generator().manual_seed(seed)
    R = len(lengths)
    pages_per = [-(-n // page) for n in lengths]
    num_pages = sum(pages_per) + 3
    perm = torch.randperm(num_pages, generator=g).tolist()
    table = torch.full((R, max(pages_per) + 1), -1, dtype=torch.int32)
    cache = (torch.randn(num_pages, 1, G, page, d + dv, generator=g)).to(dtype)
    rows = {}
    at = 0
    for r, n in enumerate(lengths):
        table[r, :pages_per[r]] = torch.tensor(perm[at:at + pages_per[r]], dtype=torch.int32)
        at += pages_per[r]
        rows[r] = torch.stack([cache[int(table[r, j // page]), 0, :, j % page] for j in range(n)]).double()      # [n, G, d + dv]
    T = sum(new)
    q = (torch.randn(T, H, d, generator=g)).to(dtype).double()
    pos, treq = [], []
    for r, (n, k) in enumerate(zip(lengths, new)):
        pos += list(range(n - k, n))
        treq += [r] * k
    scale = 0.35
    if sharpen:
        for t, j in sharpen.items():
            for h in range(H):
                key = rows[treq[t]][j, h // (H // G), :d]
                q[t, h] = (9.0 / scale) * key / (key @ key)
        q = q.to(dtype).double()
    want = torch.zeros(T, H, dv, dtype=torch.float64)
    for t in range(T):
        keys = rows[treq[t]][: pos[t] + 1]
        seen = torch.tensor([plain.visible(pos[t], j, window or None, keep) for j in range(pos[t] + 1)])
        for h in range(H):
            kv = keys[:, h // (H // G)]
            s = (kv[:, :d] @ q[t, h]) * scale
            if cap:
                s = cap * torch.tanh(s / cap)
            s = s.masked_fill(~seen, -math.inf)
            want[t, h] = torch.softmax(s, -1) @ kv[:, d:]
    out = torch.empty(T, H * dv, dtype=dtype, device="cuda")
    if tensor_cores:
        assert kernels.window_attention_mma_supports(d, dv, H, G)
        qsl = [0]
        for k in new:
            qsl.append(qsl[-1] + k)
        kernels.window_attention_mma(_dev(q.reshape(T, H * d), dtype), out, cache.cuda(), table.cuda(), _ints(qsl), _ints(lengths),
                                     [T + 64] + [1] * (len(new) - 1), H, G, d, dv, scale, cap or 0.0, window, keep, splits=splits)
    else:
        kernels.window_attention_generic(_dev(q.reshape(T, H * d), dtype), out, cache.cuda(), table.cuda(), _ints(pos), _ints(treq),
                                         H, G, d, dv, scale, cap or 0.0, window, keep)
    return out.view(T, H, dv), want


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("decode", [False, True])
def test_one_key_stands_out_at_every_edge(dtype, decode):
    """A key whose score is made to dominate must be seen exactly when the design says so: the last key inside the
    window and the first outside, the last kept token and the first not kept, the very first token, both sides of page
    borders, the query's own key; for a query inside a prompt's portion and for a single decoded token."""
    page, window, keep, n = 8, 21, 5, 96
    pos = n - 1
    cases = [(pos - window + 1, True), (pos - window, False), (pos, True), (pos - 7, True), (pos - 8, True), (keep - 1, True),
             (keep, False), (0, True), (7, False), (8, False), (40, False)]
    for j, expected in cases:
        assert plain.visible(pos, j, window, keep) == expected
        new, t = ([1, 1], 0) if decode else ([30, 3], 29)
        got, want = _attention_case(dtype, 4, 2, 24, 12, [n, 40], new, page, 7 + j, window, keep, 25.0, sharpen={t: j})
        _close(got, want, dtype, f"query {pos} with key {j} standing out")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,d,dv,window,keep,cap", [(3, 1, 20, 36, 0, 0, 0.0), (6, 3, 64, 16, 16, 16, 10.0), (2, 2, 7, 5, 3, 1, 0.0),
                                                      (8, 2, 128, 128, 40, 0, 50.0), (1, 1, 32, 160, 1, 0, 0.0)])
def test_attention_of_many_shapes(dtype, H, G, d, dv, window, keep, cap):
    got, want = _attention_case(dtype, H, G, d, dv, [50, 1, 17, 70], [50, 1, 2, 1], 16, d + window, window, keep, cap)
    _close(got, want, dtype, "attention output")


@pytest.mark.parametrize("d,dv,H,G", [(64, 32, 4, 2), (64, 64, 8, 2), (128, 128, 2, 2), (128, 64, 6, 1), (64, 128, 4, 4), (128, 32, 2, 1)])
def test_attention_on_the_tensor_cores(d, dv, H, G):
    """The tensor-core kernel against plain attention over the same cached rows: windows that start inside and between
    key tiles, kept tokens before the window, in it and none, requests of one token beside long portions, a launch
    sized for more tiles than the batch has (a captured step's upper bound); and a key made to stand out at the
    window's and the kept tokens' edges."""
    dtype = torch.bfloat16
    for window, keep, cap in ((0, 0, 0.0), (70, 9, 30.0), (64, 0, 0.0), (200, 130, 15.0), (5, 70, 0.0)):
        got, want = _attention_case(dtype, H, G, d, dv, [300, 1, 97, 210], [300, 1, 40, 3], 16, d + dv + window, window, keep, cap,
                                    tensor_cores=True)
        _close(got, want, dtype, f"attention output with window {window} keeping {keep}")
    window, keep, n = 70, 9, 260
    for j in (n - 1 - window + 1, n - 1 - window, keep - 1, keep, 0, 63, 64, n - 1):
        got, want = _attention_case(dtype, H, G, d, dv, [n, 50], [100, 2], 16, j, window, keep, 25.0, sharpen={99: j}, tensor_cores=True)
        _close(got, want, dtype, f"query {n - 1} with key {j} standing out")


@pytest.mark.parametrize("splits", [2, 3, 8])
def test_decode_steps_share_a_window_over_several_ctas(splits):
    """Single decoded tokens whose key tiles are split over CTAs and merged: windows longer and shorter than the context,
    more splits than a request has tiles (CTAs without a tile), a key made to stand out in the first, a middle and the
    last split and among the kept tokens."""
    dtype = torch.bfloat16
    for window, keep, cap in ((0, 0, 0.0), (300, 6, 30.0), (40, 100, 0.0)):
        got, want = _attention_case(dtype, 8, 2, 64, 64, [700, 1, 97, 333], [1, 1, 1, 1], 16, 5 + window, window, keep, cap,
                                    tensor_cores=True, splits=splits)
        _close(got, want, dtype, f"decode with window {window} keeping {keep} over {splits} splits")
    n, window, keep = 640, 300, 6
    for j in (n - window, n - window - 1, keep - 1, keep, 400, n - 65, n - 1):
        got, want = _attention_case(dtype, 4, 2, 128, 64, [n, 20], [1, 1], 16, j, window, keep, 25.0, sharpen={0: j}, tensor_cores=True, splits=splits)
        _close(got, want, dtype, f"query {n - 1} with key {j} standing out over {splits} splits")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rotation_unit_norm_value_mixing_and_cache_write(dtype):
    from cuinfer_b200 import kernels

    g = torch.Generator().manual_seed(3)
    T, H, G, d, dv, dims, page = 9, 4, 2, 10, 6, 6, 4
    rows = torch.randn(T, (H + G) * d + G * dv + 3, generator=g).to(dtype).double()
    v_first = torch.randn(T, G * dv, generator=g).to(dtype).double()
    lam = torch.tensor([0.3125], dtype=torch.float64)
    positions = [0, 1, 2, 3, 1000, 1001, 70000, 5, 6]
    slots = [7, 2, 3, -1, 0, 1, 11, 10, 5]
    freqs = plain.rotary_frequencies(250.0, dims, {"factor": 3.0, "low": 1.0, "high": 2.0, "original": 40})
    cache = torch.zeros(3, 1, G, page, d + dv, dtype=dtype, device="cuda")
    dev = _dev(rows, dtype)
    kernels.window_attention_prep(dev, _ints(positions), _ints(slots), torch.tensor(freqs, dtype=torch.float32).cuda(), dims, 1e-5,
                                  H, G, d, dv, _dev(v_first, dtype), _dev(lam, dtype), cache)
    # the design takes the angle in 32 bits: position times frequency, both as float32; the plain rotation gets those
    # angles by way of "positions" 1 and "frequencies" per token
    f32 = torch.tensor(freqs, dtype=torch.float32)

    def rotated(x):
        out = torch.empty_like(x)
        for t in range(T):
            angles = (torch.tensor(float(positions[t]), dtype=torch.float32) * f32).double().tolist()
            out[t] = plain.rotate_pairs(x[t:t + 1], torch.ones(1), angles)[0]
        return out

    q = plain.rms(rotated(rows[:, :H * d].view(T, H, d)), 1e-5)
    k = plain.rms(rotated(rows[:, H * d:(H + G) * d].view(T, G, d)), 1e-5)
    v = (1 - lam) * rows[:, (H + G) * d:(H + G) * d + G * dv].view(T, G, dv) + lam * v_first.view(T, G, dv)
    _close(dev[:, :H * d].view(T, H, d), q, dtype, "queries")
    for t in range(T):
        if slots[t] < 0:
            continue
        got = cache[slots[t] // page, 0, :, slots[t] % page]
        _close(got[:, :d], k[t], dtype, f"key of token {t} at position {positions[t]}")
        _close(got[:, d:], v[t], dtype, f"mixed value of token {t}")
    flat = cache.permute(0, 3, 1, 2, 4).reshape(-1, G, d + dv)
    assert float(flat[[4, 6, 8, 9]].abs().max()) == 0.0, "a token without slot wrote somewhere"


def _portioned(lengths_by_request, cuts):
    """Rows of several requests laid out for steps: ``cuts[s][r]`` tokens of request r in step s."""
    done = [0] * len(lengths_by_request)
    for step in cuts:
        yield [(r, done[r], done[r] + n) for r, n in enumerate(step) if n], done
        for r, n in enumerate(step):
            done[r] += n


def _select(total, start, size):
    """[size, total]: a projection that picks the columns start..start+size-1."""
    m = torch.zeros(size, total, dtype=torch.float64)
    m[torch.arange(size), start + torch.arange(size)] = 1.0
    return m


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,d,dv", [(3, 20, 12), (1, 40, 72), (2, 64, 128), (2, 130, 33)])
def test_matrix_memory_through_portions_and_slots(dtype, H, d, dv):
    """Two requests cut differently (down to single tokens), slots that are not in order, a padding request without a
    slot; compared with the plain recurrence over each whole sequence.  The plain side reads the same projected rows
    (rounded as the engine stores them) through projections that pick columns."""
    from cuinfer_b200 import kernels

    g = torch.Generator().manual_seed(d)
    lengths = [37, 23]
    C = 2 * H * d + 2 * H * dv
    feats = []
    for n in lengths:
        rows = torch.cat([torch.randn(n, 2 * H * d, generator=g) * 1.5, torch.randn(n, 2 * H * dv, generator=g)], dim=1).to(dtype).double()
        feats.append(torch.cat([rows, (torch.randn(n, 2 * H, generator=g) * 2).float().double()], dim=1))
    total = C + 2 * H
    w = {"q": _select(total, 0, H * d), "k": _select(total, H * d, H * d), "v": _select(total, 2 * H * d, H * dv),
         "g": _select(total, 2 * H * d + H * dv, H * dv), "i": _select(total, C, H), "f": _select(total, C + H, H),
         "i.b": torch.randn(H, generator=g).bfloat16().double(), "f.b": (2 + torch.randn(H, generator=g)).bfloat16().double(),
         "norm": (1 + 0.1 * torch.randn(H * dv, generator=g)).bfloat16().double(), "o": torch.eye(H * dv, dtype=torch.float64)}
    cfg = {"heads": H, "dim": d, "vdim": dv, "gate_cap": 6.0}
    want = [plain.mlstm_mixer(f, w, cfg, 1e-5) for f in feats]
    state = torch.zeros(5, H, d * dv + d + 1, dtype=torch.float32, device="cuda")
    state[3] = 7.0                                     # a slot nobody owns must stay as it is
    slots = [4, 1]
    got = [torch.zeros(n, H * dv, dtype=torch.float64) for n in lengths]
    cuts = [[5, 0], [1, 23], [1, 0], [30, 0]]
    for spans, _done in _portioned(lengths, cuts):
        x = torch.cat([feats[r][a:b] for r, a, b in spans])
        qsl = [0]
        for r, a, b in spans:
            qsl.append(qsl[-1] + b - a)
        qsl.append(qsl[-1])                            # a padding request: no tokens, no slot
        dev = _dev(x[:, :C], dtype)
        o = torch.empty(x.shape[0], H * dv, dtype=torch.float32, device="cuda")
        kernels.mlstm_scan(dev[:, :H * d], dev[:, H * d:2 * H * d], dev[:, 2 * H * d:2 * H * d + H * dv], _dev(x[:, C:], torch.float32),
                           _dev(w["i.b"], dtype), _dev(w["f.b"], dtype), 6.0, d ** -0.5, state, _ints(qsl), _ints([slots[r] for r, _, _ in spans] + [-1]),
                           o, H, d, dv)
        out = torch.empty(x.shape[0], H * dv, dtype=dtype, device="cuda")
        kernels.head_rms_gate(o, dev[:, 2 * H * d + H * dv:], _dev(w["norm"], dtype), 1e-5, False, out, H, dv)
        at = 0
        for r, a, b in spans:
            got[r][a:b] = out[at:at + b - a].double().cpu()
            at += b - a
    for r in range(2):
        _close(got[r], want[r], dtype, f"request {r}", tol=1e-4 if dtype == torch.float32 else 2e-2)
    assert float((state[3] - 7.0).abs().max()) == 0.0 and float(state[0].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,d,dv,K", [(4, 2, 12, 20, 4), (2, 2, 32, 32, 1), (6, 3, 64, 40, 3), (1, 1, 100, 64, 2)])
def test_delta_rule_through_portions_and_slots(dtype, H, G, d, dv, K):
    """As above for the gated delta rule; portions shorter than the convolution (one and two tokens) continue from the
    convolution's state."""
    from cuinfer_b200 import kernels

    g = torch.Generator().manual_seed(d + K)
    lengths = [37, 23]
    C = 2 * G * d + H * dv
    feats = []
    for n in lengths:
        rows = torch.randn(n, C + H * dv, generator=g).to(dtype).double()
        feats.append(torch.cat([rows, torch.randn(n, 2 * H, generator=g).float().double()], dim=1))
    total = C + H * dv + 2 * H
    w = {"q": _select(total, 0, G * d), "k": _select(total, G * d, G * d), "v": _select(total, 2 * G * d, H * dv),
         "g": _select(total, C, H * dv), "b": _select(total, C + H * dv, H), "a": _select(total, C + H * dv + H, H),
         "q.conv": torch.randn(G * d, K, generator=g) * 0.6, "k.conv": torch.randn(G * d, K, generator=g) * 0.6,
         "v.conv": torch.randn(H * dv, K, generator=g) * 0.6, "A_log": torch.randn(H, generator=g) - 1, "dt_bias": torch.randn(H, generator=g),
         "norm": 1 + 0.1 * torch.randn(dv, generator=g), "o": torch.eye(H * dv)}
    w = {k: v.bfloat16().double() for k, v in w.items()}
    cfg = {"heads": H, "kv_heads": G, "dim": d, "vdim": dv, "conv": K}
    memory = torch.zeros(5, H, d * dv, dtype=torch.float32, device="cuda")
    conv = torch.zeros(5, max(K - 1, 1), C, dtype=torch.float32, device="cuda")
    slots = [2, 0]
    got = [torch.zeros(n, H * dv, dtype=torch.float64) for n in lengths]
    taps = torch.cat([w["q.conv"], w["k.conv"], w["v.conv"]])
    cuts = [[1, 0], [2, 23], [1, 0], [1, 0], [32, 0]]
    for spans, _done in _portioned(lengths, cuts):
        x = torch.cat([feats[r][a:b] for r, a, b in spans])
        qsl, treq = [0], []
        for i, (r, a, b) in enumerate(spans):
            qsl.append(qsl[-1] + b - a)
            treq += [i] * (b - a)
        dev = _dev(x[:, :C + H * dv], dtype)
        qkv = torch.empty(x.shape[0], C, dtype=torch.float32, device="cuda")
        sl = _ints([slots[r] for r, _, _ in spans])
        kernels.delta_prep(dev, _dev(taps, dtype), conv, _ints(qsl), _ints(treq), sl, G, H, d, dv, 1e-6, d ** -0.5, qkv)
        o = torch.empty(x.shape[0], H * dv, dtype=torch.float32, device="cuda")
        kernels.delta_scan(qkv, _dev(x[:, C + H * dv:], torch.float32), _dev(w["A_log"], dtype), _dev(w["dt_bias"], dtype), memory,
                           _ints(qsl), sl, o, G, H, d, dv)
        out = torch.empty(x.shape[0], H * dv, dtype=dtype, device="cuda")
        kernels.head_rms_gate(o, dev[:, C:], _dev(w["norm"], dtype), 1e-5, True, out, H, dv)
        at = 0
        for r, a, b in spans:
            got[r][a:b] = out[at:at + b - a].double().cpu()
            at += b - a
    for r in range(2):
        want = plain.delta_mixer(feats[r], w, cfg, 1e-5)
        _close(got[r], want, dtype, f"request {r}", tol=1e-4 if dtype == torch.float32 else 2e-2)


# ---- other sizes, drawn at random ---------------------------------------------------------------------------------------
def _random_config(seed):
    """A small configuration whose every size, count, constant and the order of its layers is drawn: ones, absent parts
    (no window, no cap, no rotation, no scaling, no feed-forward, no per-layer token input); from seed 10 on every size
    is odd or at least no multiple of eight."""
    import random

    rnd = random.Random(seed)
    odd = seed >= 10
    pick = lambda even_sizes, odd_sizes: rnd.choice(odd_sizes if odd else even_sizes)      # noqa: E731
    width = pick([24, 40, 56, 64, 100], [37, 50, 66, 98, 131])
    vocab = pick([33, 64, 131], [31, 77, 257])
    mix_heads, mix_vdim = pick([1, 2, 3], [1, 2, 5]), pick([4, 8, 20, 32], [3, 7, 10, 33])      # layers that mix values agree in these

    def feed_forward():
        kind = rnd.choice(["dense", "moe", "moe", None])
        if kind == "dense":
            return {"kind": "dense", "ff": pick([16, 40, 96], [15, 41, 99])}
        if kind == "moe":
            experts = rnd.randint(2, 6)
            return _moe(experts, rnd.randint(1, experts), pick([8, 16, 32], [7, 18, 33]), rnd.choice([0.5, 1.0, 7.0]))
        return None

    layers = []
    for _ in range(rnd.randint(2, 5)):
        kind = rnd.choice(["attention", "attention", "mlstm", "delta"])
        if kind == "attention":
            v_mix = rnd.random() < 0.6
            kv = mix_heads if v_mix else pick([1, 2, 4], [1, 3, 5])
            dim = pick([8, 12, 16, 20, 32, 64], [6, 7, 9, 14, 22, 50])
            rot = None
            if rnd.random() < 0.8:
                rot = {"base": rnd.choice([50.0, 1e4, 1e6]), "dims": rnd.choice([2, 4, dim // 4 * 2, dim // 2 * 2])}
                if rnd.random() < 0.5:
                    rot["scaling"] = {"factor": rnd.choice([2.0, 8.0]), "low": 1.0, "high": rnd.choice([2.0, 4.0]), "original": rnd.choice([16, 64, 512])}
            window = pick([None, 1, 3, 8, 16, 33, 64], [None, 1, 2, 7, 15, 31, 65])
            layers.append(_attention(kv * pick([1, 2, 4], [1, 2, 3]), kv, dim, mix_vdim if v_mix else pick([4, 8, 16, 20, 32], [5, 9, 17, 40]),
                                     rnd.choice([0.5, 1.0, 2.0]) / math.sqrt(dim), window=window, keep=pick([0, 1, 4, 20], [0, 1, 3, 17]), rot=rot,
                                     softcap=rnd.choice([None, 5.0, 30.0]), v_mix=v_mix, mlp=feed_forward()))
        elif kind == "mlstm":
            layers.append({"type": "mlstm", "mixer": {"heads": rnd.randint(1, 4), "dim": pick([4, 12, 16, 33, 48], [3, 11, 31, 65, 129]),
                                                      "vdim": pick([8, 16, 24, 40], [5, 17, 33, 70]), "gate_cap": rnd.choice([5.0, 15.0])}, "mlp": feed_forward()})
        else:
            kv = rnd.randint(1, 3)
            layers.append({"type": "delta", "mixer": {"heads": kv * pick([1, 2], [1, 3]), "kv_heads": kv, "dim": pick([4, 8, 16, 24, 40], [3, 9, 33, 70]),
                                                      "vdim": pick([8, 12, 16, 32], [5, 13, 31, 66]), "conv": rnd.randint(1, 5)}, "mlp": feed_forward()})
    return _config(vocab, width, layers, side=pick([None, 2, 6, 10], [None, 1, 5, 9]), eps=rnd.choice([1e-6, 1e-5, 1e-3])), pick([16, 32], [16, 32, 64])


@pytest.mark.parametrize("seed", range(16))
def test_configurations_drawn_at_random(seed, tmp_path):
    cfg, page = _random_config(seed)
    tensors = plain.random_model(cfg, 100 + seed)
    t64 = {k: v.double() for k, v in tensors.items()}
    requests = _requests(cfg, [1, 23, 70, 9], seed=30 + seed)
    steps = traces.mixed(requests, max_live=3, sizes=(5, 2, 11, 3))
    refs = {}
    for rid, toks in requests.items():
        assert plain.router_margin(cfg, t64, list(toks)) > 0.03, "the drawn routers must not rest on a close call"
        refs[rid] = plain.forward(cfg, t64, list(toks)).numpy()
    for dtype in ("float32", "bfloat16"):
        folder = _write(str(tmp_path / dtype), cfg, tensors, dtype)
        out = str(tmp_path / f"out_{dtype}")
        traces.replay_in_process(folder, dtype, steps, out, traces.live_token_peak(steps), page, max_live=4)
        got = traces.collect(steps, out, cfg["vocab"])
        whole_steps = traces.whole(requests)
        whole_out = str(tmp_path / f"whole_{dtype}")
        traces.replay_in_process(folder, dtype, whole_steps, whole_out, traces.live_token_peak(whole_steps), page)
        whole = traces.collect(whole_steps, whole_out, cfg["vocab"])
        errors = []
        for rid, toks in requests.items():
            for pos, row in sorted(got[rid].items()):
                assert np.isfinite(row).all()
                errors.append((_row_error(row, refs[rid][pos]), rid, pos))
                if dtype == "float32":
                    cut = _row_error(row, whole[rid][pos].astype(np.float64))
                    assert cut <= CUT_TOLERANCE[dtype], f"configuration {seed}: request {rid} position {pos} depends on the cut ({cut:.3e}): {json.dumps(cfg)}"
        # float32 is held row by row, but for the few positions that the design itself conditions badly (see _check); the
        # bfloat16 run of these very narrow layers is held by its median row, which a wrong shape or kernel choice would move
        ranked = sorted(errors)
        if dtype == "float32":
            assert ranked[int(0.97 * len(ranked))][0] <= TOLERANCE[dtype] and ranked[-1][0] <= 25 * TOLERANCE[dtype], \
                f"configuration {seed}: request {ranked[-1][1]} position {ranked[-1][2]} (error {ranked[-1][0]:.3e}): {json.dumps(cfg)}"
        else:
            assert ranked[len(ranked) // 2][0] <= 0.05, f"configuration {seed} in bfloat16: median row error {ranked[len(ranked) // 2][0]:.3e}: {json.dumps(cfg)}"
