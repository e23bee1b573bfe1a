"""Kudadra on the GPU: every new kernel alone against the plain functions, then the model through the engine's own step
function, cache manager, scheduler and replay tool against the plain implementation, on four tiny configurations."""
import math
import os
import random

import numpy as np
import pytest
import torch

from lightllm_b200 import Engine, EngineCore, EngineOptions, StepEntry
from lightllm_b200.csrc import ops
from tests.kudadra_configs import CONFIGS, PAGE_SIZE, config, random_weights, write_model
from tests.plain import kudadra_plain as K
from tests.tolerances import FLOAT32_ATOL, KUDADRA_BF16_WORST_REL, logits_std, record
from tests.trace_util import Trace, compare_with_plain, run_trace

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def dev(t, dtype=None):
    return t.to(DEV, dtype=dtype).contiguous()


def close(got, want, dtype, what, rel=None):
    """float32: 2e-5 of the result's scale; bfloat16: a few roundings of 2^-9."""
    scale = float(want.abs().max()) + 1e-6
    tol = (2e-5 if dtype == "float32" else 2.5e-2) * scale if rel is None else rel * scale
    err = float((got.double().cpu() - want.double()).abs().max())
    assert err <= tol, f"{what}: max |diff| {err:.3e} > {tol:.3e}"


# ---------------------------------------------------------------------------------------------------------------------
# kernels alone
# ---------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("D", [44, 320, 1500, 5000])
@pytest.mark.parametrize("wdtype", ["float32", "bfloat16"])
def test_layer_norm_kernel(D, wdtype):
    torch.manual_seed(D)
    x = torch.randn(13, D) * 3 + 1.5
    w, b = (1 + 0.1 * torch.randn(D)).to(DT[wdtype]), (0.1 * torch.randn(D)).to(DT[wdtype])
    want = K.plain_layer_norm(x.double(), w.double(), b.double(), 1e-5)
    out = torch.empty(13, D, device=DEV)
    ops.layernorm(dev(x), dev(w), dev(b), 1e-5, out)
    close(out, want, "float32", "layer norm")
    rows = torch.tensor([12, 0, 5], dtype=torch.int32)
    out = torch.empty(3, D, device=DEV, dtype=DT[wdtype])
    ops.layernorm(dev(x), dev(w), dev(b), 1e-5, out, rows=dev(rows))
    close(out, want[rows.long()], wdtype, "layer norm of rows")
    acc = torch.randn(13, D)
    out = dev(acc)
    copy = torch.empty(13, D, device=DEV, dtype=torch.bfloat16)
    ops.layernorm(dev(x), dev(w), dev(b), 1e-5, out, accumulate=True, copy=copy)
    close(out, acc.double() + want, "float32", "layer norm added into the stream")
    assert torch.equal(copy, out.bfloat16())          # the new stream once more, in bfloat16


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_gated_activation_kernel(dtype):
    torch.manual_seed(2)
    x = (torch.randn(7, 2 * 37) * 3).to(DT[dtype])
    g, u = x[:, 0::2].double(), x[:, 1::2].double()
    for limit in (0.5, 1.0, 7.0):
        gg, uu = g.clamp(max=limit), u.clamp(-limit, limit)
        want = gg * torch.sigmoid(1.702 * gg) * (uu + 1.0)
        out = torch.empty(7, 37, device=DEV, dtype=DT[dtype])
        ops.glu_act(dev(x), out, ops.GLU_CLAMPED_SWISH, 1.702, limit, 1.0)
        close(out, want, dtype, f"clamped gate, limit {limit}", rel=None if dtype == "float32" else 5e-3)
    out = torch.empty(7, 37, device=DEV, dtype=DT[dtype])
    ops.glu_act(dev(x), out, ops.GLU_SILU)
    close(out, g * torch.sigmoid(g) * u, dtype, "silu gate", rel=None if dtype == "float32" else 5e-3)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,hd,vd,rot", [(4, 2, 12, 20, 6), (3, 3, 64, 64, 64), (2, 1, 16, 8, 0), (8, 2, 64, 64, 32)])
def test_norm_rotation_and_cache_write_from_a_fused_projection(dtype, H, G, hd, vd, rot):
    torch.manual_seed(H * hd)
    T, extra = 9, 5
    C = H * hd + G * hd + G * vd + extra
    src = torch.randn(T, C).to(DT[dtype])
    qw, kw = 1 + 0.2 * torch.randn(H * hd), 1 + 0.2 * torch.randn(G * hd)
    pos = torch.tensor([0, 1, 2, 3, 700, 701, 9, 10, 11], dtype=torch.int32)
    slots = torch.tensor([5, 4, 3, 2, 1, 0, 20, 21, -1], dtype=torch.int32)
    inv = (1.0 / 10000.0 ** (torch.arange(0, rot, 2, dtype=torch.float64) / max(rot, 1))).float()
    s = src.double()
    q = K.plain_rotate(K.plain_rms(s[:, :H * hd], 1e-5, qw.double()).view(T, H, hd), pos, rot, 10000.0)
    k = K.plain_rotate(K.plain_rms(s[:, H * hd:(H + G) * hd], 1e-5, kw.double()).view(T, G, hd), pos, rot, 10000.0)
    v = s[:, (H + G) * hd:(H + G) * hd + G * vd].view(T, G, vd)
    q_out = torch.empty(T, H * hd, device=DEV, dtype=DT[dtype])
    kc = torch.full((24, G, hd), float("nan"), device=DEV, dtype=DT[dtype])
    vc = torch.full((24, G, vd), float("nan"), device=DEV, dtype=DT[dtype])
    ops.qkv_prepare(dev(src), 0, H * hd, (H + G) * hd, H, G, hd, vd, dev(pos), dev(slots), q_out, kc, vc, dev(qw), dev(kw),
                    1e-5, dev(inv) if rot else None, rot, False)
    close(q_out.view(T, H, hd), q, dtype, "q")
    live = slots >= 0
    close(kc[slots[live].long()], k[live], dtype, "k rows")
    close(vc[slots[live].long()], v[live], dtype, "v rows", rel=0.0)
    untouched = torch.ones(24, dtype=torch.bool)
    untouched[slots[live].long()] = False
    assert torch.isnan(kc[untouched.to(DEV)].float()).all()          # the token without a slot wrote nowhere


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_contraction_per_head(dtype):
    torch.manual_seed(4)
    for T, H, i, o, off in ((1, 3, 12, 28, 0), (37, 5, 40, 16, 7), (16, 1, 128, 48, 0)):
        x = torch.randn(T, off + H * i + 3).to(DT[dtype])
        w = (torch.randn(H, o, i) / i ** 0.5).to(DT[dtype])
        want = torch.einsum("thi,hoi->tho", x[:, off:off + H * i].double().view(T, H, i), w.double()).reshape(T, H * o)
        out = torch.empty(T, H * o, device=DEV, dtype=DT[dtype])
        ops.head_linear(dev(x), off, dev(w), out)
        close(out, want, dtype, f"per-head contraction {T}x{H}x{i}x{o}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_head_gates(dtype):
    torch.manual_seed(5)
    T, H, hd = 6, 3, 20
    x = torch.randn(T, H * hd) * 2
    wide = torch.randn(T, 11 + H * hd).to(DT[dtype])               # the gate's input is a column range of a wider tensor
    z = wide[:, 11:].double()
    xa = x.to(DT[dtype])
    out = torch.empty(T, H * hd, device=DEV, dtype=DT[dtype])
    ops.head_gate(dev(xa), dev(wide)[:, 11:], out, H, hd, False, "sigmoid")
    close(out, xa.double() * torch.sigmoid(z), dtype, "sigmoid gate, element by element", rel=None if dtype == "float32" else 6e-3)
    ops.head_gate(dev(xa), dev(wide)[:, 11:11 + H], out, H, hd, True, "sigmoid")
    want = (xa.double().view(T, H, hd) * torch.sigmoid(z[:, :H])[:, :, None]).reshape(T, -1)
    close(out, want, dtype, "sigmoid gate, one number a head", rel=None if dtype == "float32" else 6e-3)
    ops.head_gate(dev(x), dev(wide)[:, 11:], out, H, hd, False, "silu", unit_rms=True, eps=1e-5)       # float32 in
    want = K.plain_rms(x.double().view(T, H, hd), 1e-5).reshape(T, -1) * z * torch.sigmoid(z)
    close(out, want, dtype, "unit-rms heads times silu gate", rel=None if dtype == "float32" else 6e-3)


def plain_retention_core(q, k, v, decay, k_scale, rot, base, pos0, S0):
    """o_t and the final state from already projected q, k [T, H, d], v [T, H, e], in float64."""
    T, H, d = q.shape
    pos = torch.arange(pos0, pos0 + T)
    q, k = K.plain_rotate(q, pos, rot, base), K.plain_rotate(k, pos, rot, base) * k_scale
    S = S0.clone()
    out = torch.zeros(T, H, v.shape[-1], dtype=torch.float64)
    for t in range(T):
        for h in range(H):
            S[h] = decay[h] * S[h] + torch.outer(k[t, h], v[t, h])
            out[t, h] = S[h].T @ q[t, h]
    return out, S


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("chunk", [0, 5, 16])
@pytest.mark.parametrize("H,d,e,rot", [(3, 12, 20, 8), (2, 64, 64, 64), (2, 128, 64, 64), (1, 256, 40, 0), (4, 16, 300, 16)])
def test_retention_kernel_over_spans_and_slots(dtype, H, d, e, rot, chunk):
    """Three requests in one launch: one from its first token, one that continues from a state another launch left (in
    a slot that a finished request used before), one single token; then the same sequences cut differently."""
    torch.manual_seed(d + e)
    base = 1000.0
    decay = [0.5, 0.9, 0.99, 1.0][:H]
    lens = {"a": 37, "b": 21, "c": 18}
    C = 2 * H * d + H * e + 3
    proj = {r: (torch.randn(n, C) * 0.7).to(DT[dtype]) for r, n in lens.items()}
    inv = dev((1.0 / base ** (torch.arange(0, rot, 2, dtype=torch.float64) / max(rot, 1))).float()) if rot else None
    dec = dev(torch.tensor(decay))
    state = torch.full((4, H, d, e), float("nan"), device=DEV)          # a slot's old content must never be read at position 0

    def run(parts):
        """parts: (request, slot, from, to).  With ``chunk`` the spans are cut into pieces of so many tokens that run
        side by side (their contributions to the state are scanned in between)."""
        rows = torch.cat([proj[r][a:b] for r, _, a, b in parts])
        o = torch.empty(rows.shape[0], H * e, device=DEV)
        starts = np.cumsum([0] + [b - a for _, _, a, b in parts])[:-1]
        i32 = lambda xs: dev(torch.tensor(list(xs), dtype=torch.int32))
        pieces = None
        if chunk:
            counts = [-(-(b - a) // chunk) for _, _, a, b in parts]
            item_span = [i for i, n in enumerate(counts) for _ in range(n)]
            item_c = [c for n in counts for c in range(n)]
            pieces = (i32(item_span), i32(item_c), i32(np.cumsum([0] + counts)[:-1]), len(item_span), chunk)
        ops.retention(dev(rows), 0, H * d, 2 * H * d, i32(starts), i32(b - a for _, _, a, b in parts),
                      i32(a for _, _, a, _ in parts), i32(s for _, s, _, _ in parts), len(parts), H, d, e, dec, inv, rot,
                      False, d ** -0.5, state, o, pieces=pieces)
        out, at = {}, 0
        for r, _, a, b in parts:
            out[(r, a, b)] = o[at:at + b - a].cpu()
            at += b - a
        return out

    want = {}
    for r, n in lens.items():
        p = proj[r].double()
        want[r] = plain_retention_core(p[:, :H * d].view(n, H, d), p[:, H * d:2 * H * d].view(n, H, d),
                                       p[:, 2 * H * d:2 * H * d + H * e].view(n, H, e), decay, d ** -0.5, rot, base, 0,
                                       torch.zeros(H, d, e, dtype=torch.float64))
    got = {}
    got.update(run([("a", 2, 0, 17), ("c", 0, 0, 18)]))                  # c ends here; its slot 0 is used again below
    got.update(run([("a", 2, 17, 18), ("b", 0, 0, 2)]))                  # a single token beside a portion of two
    got.update(run([("b", 0, 2, 21), ("a", 2, 18, 37)]))
    for (r, a, b), o in got.items():
        close(o.view(b - a, H, e), want[r][0][a:b], "float32", f"retention {r}[{a}:{b}]", rel=2e-5)
    close(state[2], want["a"][1], "float32", "state of a", rel=2e-5)
    close(state[0], want["b"][1], "float32", "state of b", rel=2e-5)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", ["values wider", "values narrower", "values in the key rows", "plain"])
def test_attention_kernel_with_sinks_and_value_widths(dtype, shape):
    """The CUDA-core attention over shuffled pages: a portion whose queries start at position 300, in tiles of rows and
    row by row with the keys in pieces, and a single token, with and without sinks and a window."""
    torch.manual_seed(7)
    H, G, hd = 6, 2, 24
    vd = {"values wider": 40, "values narrower": 10, "values in the key rows": hd, "plain": hd}[shape]
    if shape == "values in the key rows":
        G = 1
    page, npages, n = 8, 64, 333
    pages = torch.randperm(npages)[: -(-n // page)].to(torch.int32)
    k = (torch.randn(n, G, hd)).to(DT[dtype])
    v = k if shape == "values in the key rows" else torch.randn(n, G, vd).to(DT[dtype])
    kc = torch.full((npages * page, G, hd), float("nan"), dtype=DT[dtype])
    vc = torch.full((npages * page, G, vd), float("nan"), dtype=DT[dtype])
    slot = pages[torch.arange(n) // page].long() * page + torch.arange(n) % page
    kc[slot], vc[slot] = k, v
    kc_d = dev(kc)
    vc_d = kc_d if shape == "values in the key rows" else dev(vc)
    sinks = torch.tensor([0.0, 3.0, -2.0, 6.0, 1.0, 9.0])
    bt = dev(pages.view(1, -1))
    i32 = lambda *xs: dev(torch.tensor(xs, dtype=torch.int32))
    for start, rows, bq, nsplit in ((300, 33, 4, 1), (300, 33, 1, 3), (332, 1, 1, 1), (332, 1, 1, 4), (0, 20, 16, 1)):
        for window, use_sinks in ((0, True), (50, False), (7, True)):
            q = (torch.randn(rows, H, hd) * 1.5).to(DT[dtype])
            kk, vv = k.double()[: start + rows], v.double()[: start + rows]
            want = torch.zeros(rows, H, vd, dtype=torch.float64)
            for r in range(rows):
                p = start + r
                lo = max(0, p - window + 1) if window else 0
                for h in range(H):
                    s = (kk[lo:p + 1, h // (H // G)] @ q[r, h].double()) * 0.3
                    if use_sinks:
                        s = torch.cat([s, sinks[h:h + 1].double()])
                    w = torch.softmax(s, 0)[: p + 1 - lo]
                    want[r, h] = w @ vv[lo:p + 1, h // (H // G)]
            out = torch.empty(rows, H * vd, device=DEV, dtype=DT[dtype])
            tq0 = list(range(0, rows, bq))
            scratch = torch.empty(ops.attention_scratch_floats(len(tq0), H, vd, bq, nsplit), device=DEV) if nsplit > 1 else None
            ops.paged_attention_simt(dev(q).view(rows, H * hd), kc_d, vc_d, out, i32(*([0] * len(tq0))), i32(*tq0), len(tq0),
                                     i32(0), i32(rows), i32(start), bt, bt.shape[1], page, H, G, hd, window, 0.3, bq,
                                     nsplit, scratch, v_head_dim=vd, sinks=dev(sinks) if use_sinks else None)
            close(out.view(rows, H, vd), want, dtype, f"{shape}: start {start}, {rows} rows, bq {bq}, {nsplit} pieces, "
                  f"window {window}, sinks {use_sinks}", rel=None if dtype == "float32" else 1.5e-2)


@pytest.mark.parametrize("hd", [64, 128])
@pytest.mark.parametrize("window", [0, 200, 5, 129])
def test_tensor_core_attention_with_sinks_over_values_in_the_key_rows(hd, window):
    """The tcgen05 prefill kernel (whole key ranges and ranges cut into pieces that a second kernel merges) and the
    mma.sync decode kernel (pieces merged in a cluster, and through scratch): one kv head whose rows are keys and
    values at once, six query heads, sinks from negligible to dominant."""
    torch.manual_seed(hd + window)
    H, page, npages, n = 6, 16, 64, 700
    pages = torch.randperm(npages)[: -(-n // page)].to(torch.int32)
    k = torch.randn(n, 1, hd).to(torch.bfloat16)
    kc = torch.full((npages * page, 1, hd), float("nan"), dtype=torch.bfloat16)
    kc[pages[torch.arange(n) // page].long() * page + torch.arange(n) % page] = k
    kc_d, bt = dev(kc), dev(pages.view(1, -1))
    sinks = torch.tensor([-20.0, 0.0, 2.0, 4.0, 8.0, 1.0])
    i32 = lambda *xs: dev(torch.tensor(xs, dtype=torch.int32))
    scale = 0.5 / hd ** 0.5

    def plain(q, start):
        rows = q.shape[0]
        want = torch.zeros(rows, H, hd, dtype=torch.float64)
        for r in range(rows):
            p = start + r
            lo = max(0, p - window + 1) if window else 0
            for h in range(H):
                s = torch.cat([(k.double()[lo:p + 1, 0] @ q[r, h].double()) * scale, sinks[h:h + 1].double()])
                want[r, h] = torch.softmax(s, 0)[: p + 1 - lo] @ k.double()[lo:p + 1, 0]
        return want

    for start, rows, chunk in ((0, 300, None), (380, 320, 2), (690, 10, None)):
        q = torch.randn(rows, H, hd).to(torch.bfloat16)
        out = torch.empty(rows, H * hd, device=DEV, dtype=torch.bfloat16)
        # the engine's own cutting of tiles into work items
        from lightllm_b200.engine.batch import Span, StepContext
        ctx = StepContext()
        ctx.spans, ctx.device = [Span("a", 0, start, rows, 0)], DEV
        ctx.iota, ctx.zeros = i32(0), i32(0)
        ts, tq, nt, cut = ctx.attention_items(1, window, chunk, H, 296)
        ops.paged_attention_tcgen05(dev(q).view(rows, H * hd), kc_d, kc_d, out, ts, tq, nt, i32(0), i32(rows), i32(start),
                                    bt, bt.shape[1], page, H, 1, hd, window, scale, cut=cut, sinks=dev(sinks))
        ops.check_async_errors(DEV)
        close(out.view(rows, H, hd), plain(q, start), "bfloat16", f"tcgen05, start {start}, {rows} rows, pieces of {chunk}",
              rel=1.5e-2)
    for nsplit in (1, 4, 20):
        q = torch.randn(1, H, hd).to(torch.bfloat16)
        out = torch.empty(1, H * hd, device=DEV, dtype=torch.bfloat16)
        scratch = None
        if nsplit > ops.decode_mma_cluster_splits():
            scratch = torch.empty(ops.attention_scratch_floats(1, H, hd, 1, nsplit), device=DEV)
        ops.paged_decode_mma(dev(q).view(1, H * hd), kc_d, kc_d, out, i32(0), i32(0), 1, i32(0), i32(n - 1), bt, bt.shape[1],
                             page, H, 1, hd, window, scale, nsplit, scratch, sinks=dev(sinks))
        close(out.view(1, H, hd), plain(q, n - 1), "bfloat16", f"decode, {nsplit} pieces", rel=1.5e-2)


# ---------------------------------------------------------------------------------------------------------------------
# the model through the engine
# ---------------------------------------------------------------------------------------------------------------------
def make_model(tmp_path, name, dtype, seed=3, **kw):
    cfg = config(name)
    w = random_weights(cfg, seed, store=DT[dtype], **kw)
    d = write_model(cfg, w, str(tmp_path / f"kud_{name}_{seed}"))
    return d, cfg, {k: v.double() for k, v in w.items()}


def core_for(d, dtype, name, pages=64, max_seqs=4, max_tokens=1024, graphs=True):
    return EngineCore(d, EngineOptions(dtype=dtype, max_seq_len=max_tokens, max_batch_tokens=max_tokens,
                                       page_size=PAGE_SIZE[name], num_pages=pages, max_seqs=max_seqs,
                                       use_cuda_graphs=graphs))


def atol_for(name, dtype, plain):
    """float32: the largest difference of any logit, 1e-4 on logits of order one.  bfloat16: the root mean square over a
    row of logits (mean taken off), at most twice the worst that a recorded run showed, relative to the logits' spread."""
    std = logits_std(plain)
    return (FLOAT32_ATOL * max(1.0, std)) if dtype == "float32" else 2.0 * KUDADRA_BF16_WORST_REL[name] * std


def row_errors(got, plain, dtype):
    d = (got.double() - plain.double())
    if dtype == "float32":
        return d.abs().max(-1).values
    return (d - d.mean(-1, keepdim=True)).pow(2).mean(-1).sqrt()


def error(got, plain, dtype, keep=None) -> float:
    e = row_errors(got, plain, dtype)
    return float(e.max() if keep is None else e[keep].max())


def well_conditioned(toks, w, cfg, plain, tol):
    """Rows of ``plain`` that rounding cannot move far: a row is set aside (in bfloat16 only) when multiplying every
    matrix by 1 + 2^-9 N(0, 1), which is what storing it in bfloat16 does, already moves its logits by the whole
    allowed error.  This happens in a sequence's first rows under a retention layer: o_0 = (q_0 . k_0) v_0 is divided by
    its own root mean square, so a q_0 . k_0 that nearly cancels decides the SIGN of the whole row.  float32 judges
    every row."""
    g = torch.Generator().manual_seed(1)
    w2 = {k: (v * (1 + 2.0 ** -9 * torch.randn(v.shape, generator=g, dtype=v.dtype)) if v.dim() == 2 else v) for k, v in w.items()}
    moved = row_errors(K.plain_forward(toks, w2, cfg).float(), plain, "bfloat16")
    return (moved <= tol) & ~cancelling_rows(toks, w, cfg)


def cancelling_rows(toks, w, cfg, noise=0.02, moved=0.3):
    """Rows at which a retention layer's normalised output hangs on a cancellation.  o_t = sum_j a_tj v_j with
    a_tj = decay^(t-j) q_t . k_j; an error of ``noise`` (2 %: what the bfloat16 layers before it have added to the stream)
    in q_t and k_j moves a_tj by about noise |q_t| |k_j| / sqrt(dim), and a row is set aside when that moves o_t by more
    than ``moved`` of its own length.  In a sequence's first rows o_t has few terms (o_0 = (q_0 . k_0) v_0), and a q . k
    that nearly cancels then decides the sign of the whole row once it is divided by its root mean square."""
    layers = []
    K.plain_forward(toks, w, cfg, layers_out=layers)
    T = len(toks)
    bad = torch.zeros(T, dtype=torch.bool)
    x = w["embed"][torch.tensor(toks)]
    pos = torch.arange(T)
    for i, layer in enumerate(cfg["layers"]):
        if layer["type"] == "retention":
            m, W = layer["mixer"], K._sub(w, f"l{i}.mix.")
            H, d, e = m["heads"], m["dim"], m["vdim"]
            rot = m.get("rot") or {"dims": 0, "base": 1.0}
            q = K.plain_rotate((x @ W["q"].T).view(T, H, d), pos, rot["dims"], rot["base"])
            k = K.plain_rotate((x @ W["k"].T).view(T, H, d), pos, rot["dims"], rot["base"])
            v = (x @ W["v"].T).view(T, H, e)
            for h in range(H):
                decay = torch.tensor(m["decay"][h], dtype=x.dtype).pow((pos[:, None] - pos[None, :]).clamp(min=0)).tril()
                o = ((q[:, h] @ k[:, h].T) * decay) @ v[:, h]
                da = noise * decay * q[:, h].norm(dim=-1)[:, None] * k[:, h].norm(dim=-1)[None, :] / d ** 0.5
                do = (da.pow(2) @ v[:, h].norm(dim=-1).pow(2)).sqrt()
                bad |= do > moved * o.norm(dim=-1)
        x = layers[i]
    return bad


LENGTHS = {"P": [1, 2, 17, 33, 70, 150, 64, 49], "Q": [3, 40, 131, 330, 129, 520, 64, 257], "R": [1, 5, 40, 90, 33, 64, 17, 200],
           "S": [2, 9, 24, 50, 8, 100, 16, 31], "T": [1, 3, 20, 45, 16, 70, 33, 9]}


def build_trace(name, seed=11):
    cfg = config(name)
    rng = random.Random(seed)
    seqs = {f"r{i}": [rng.randrange(cfg["vocab"]) for _ in range(n)] for i, n in enumerate(LENGTHS[name])}
    all_seqs = {f"{regime}{rid}": toks for rid, toks in seqs.items() for regime in "wtpm"}
    tr = Trace(all_seqs)
    for rid in seqs:
        tr.whole(f"w{rid}")
    for rid, toks in seqs.items():
        if len(toks) > 2:
            tr.last_one_by_one(f"t{rid}", tail=40)
    for i, rid in enumerate(seqs):
        if len(seqs[rid]) > 1:
            tr.portions(f"p{rid}", [[16, 7, 2, 5, 3, 2], [2, 2, 9, 31, 4], [13, 2, 64, 3], [200, 33, 2, 129]][i % 4])
    prompt_len = {f"m{rid}": max(2, len(toks) - 12) if len(toks) > 14 else len(toks) for rid, toks in seqs.items()}
    tr.mixed([f"m{rid}" for rid in seqs], prompt_len, seed=5, sizes=(2, 3, 7, 16, 40, 130) if name == "Q" else (2, 3, 5, 7, 16))
    return tr, seqs


@pytest.mark.parametrize("name", sorted(CONFIGS))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_all_regimes(name, dtype, tmp_path):
    """Through bin/trace_run: whole prompts, the last tokens one by one, portions down to two tokens, and up to four
    live requests mixed in a pool so small that pages and state slots are used again."""
    d, cfg, w = make_model(tmp_path, name, dtype)
    tr, seqs = build_trace(name)
    once = {rid: K.plain_forward(toks, w, cfg).float() for rid, toks in seqs.items()}
    plain = {f"{regime}{rid}": lg for rid, lg in once.items() for regime in "wtpm"}
    got = run_trace(d, dtype, tr, str(tmp_path / "out"), ["--page-size", str(PAGE_SIZE[name])])
    skip = None
    if dtype != "float32":
        skip = {}
        for rid, toks in seqs.items():
            ok = well_conditioned(toks, w, cfg, once[rid], atol_for(name, dtype, once))
            for regime in "wtpm":
                skip[f"{regime}{rid}"] = set((~ok).nonzero().flatten().tolist())
        assert sum(len(v) for v in skip.values()) <= 0.05 * 4 * sum(len(t) for t in seqs.values())
    worst = compare_with_plain(tr, got, plain, atol_for(name, dtype, once), f"Kudadra {name} {dtype}", rms=dtype != "float32",
                               skip=skip)
    record(f"replay Kudadra {name} {dtype} ({len(tr.steps)} steps, pool for {tr.max_tokens} tokens)", worst, logits_std(once))


def stepwise(core, rid, toks, cuts, want_all=True):
    """Feed ``toks`` in portions of the given sizes (the rest one by one); returns logits of every position."""
    core.open(rid)
    rows, at, i = [], 0, 0
    while at < len(toks):
        c = min(cuts[i], len(toks) - at) if i < len(cuts) else 1
        rows.append(core.step([StepEntry(rid, toks[at:at + c], list(range(c)))]).float().cpu())
        at += c
        i += 1
    core.close(rid)
    return torch.cat(rows)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["P", "Q"])
def test_sharp_attention_sees_far_keys_window_edges_and_the_sink(tmp_path, name, dtype):
    """q and k scaled up so that single keys carry a row's attention: a key that is lost (far back, at a page's border,
    just inside a window) or kept too long (just outside) moves the logits by far more than rounding.  Prompt in
    portions that end inside pages and windows, then 60 tokens one by one, so that windows pass over decoded tokens."""
    d, cfg, w = make_model(tmp_path, name, dtype, seed=8, sharp=4.0)
    rng = random.Random(2)
    n = 420 if name == "Q" else 200
    toks = [rng.randrange(cfg["vocab"]) for _ in range(n)]
    plain = K.plain_forward(toks, w, cfg).float()
    core = core_for(d, dtype, name)
    got = stepwise(core, "a", toks, [129, 2, 150 - 131, 31, 2, 64] if name == "Q" else [9, 2, 16, 38, 2, 70])
    keep = None if dtype == "float32" else well_conditioned(toks, w, cfg, plain, atol_for(name + " sharp", dtype, plain))
    err = error(got, plain, dtype, keep)
    record(f"sharp Kudadra {name} {dtype}", err, logits_std(plain))
    assert err <= atol_for(name + " sharp", dtype, plain) and (keep is None or keep.float().mean() > 0.95)
    core.runner.check_device_errors()
    # the plain implementation itself shows what a one-off window or a missing sink would cost here
    # (sharp scores dwarf the sinks, whose share is above rounding in float32 only; test_heavy_sinks has them large)
    for edit in ("window", "sink") if dtype == "float32" else ("window",):
        cfg2 = config(name)
        for layer in cfg2["layers"]:
            if edit == "window" and layer["type"] == "attention":
                layer["mixer"]["mask"]["size"] += 1
        w2 = dict(w)
        if edit == "sink":
            for k in w2:
                if k.endswith("sink"):
                    w2[k] = w2[k] - 30.0
        off = error(K.plain_forward(toks, w2, cfg2).float(), plain, dtype)
        print(f"{edit} off by one or left out: {off:.3e}; allowed: {atol_for(name + ' sharp', dtype, plain):.3e}")
        assert off > 1.5 * atol_for(name + " sharp", dtype, plain), (edit, off)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_heavy_sinks(tmp_path, dtype):
    """Sinks of +6: they hold most of every head's softmax mass, in prompts and in decoding."""
    d, cfg, w = make_model(tmp_path, "S", dtype, seed=9, sink=6.0)
    rng = random.Random(3)
    toks = [rng.randrange(cfg["vocab"]) for _ in range(90)]
    plain = K.plain_forward(toks, w, cfg).float()
    got = stepwise(core_for(d, dtype, "S"), "a", toks, [40, 3, 17])
    record(f"Kudadra S {dtype} heavy sinks", error(got, plain, dtype), logits_std(plain))
    assert error(got, plain, dtype) <= atol_for("S", dtype, plain)
    w2 = {k: (v - 30.0 if k.endswith("sink") else v) for k, v in w.items()}
    assert error(K.plain_forward(toks, w2, cfg).float(), plain, dtype) > 5 * atol_for("S", dtype, plain)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["P", "R"])
def test_prefill_equals_token_by_token_and_long_decoding(tmp_path, name, dtype):
    """A whole prompt in one step against the same tokens one by one from the first (300 single steps: the recurrent
    state is carried through every one, windows slide over decoded tokens only)."""
    d, cfg, w = make_model(tmp_path, name, dtype, seed=5)
    rng = random.Random(4)
    toks = [rng.randrange(cfg["vocab"]) for _ in range(300)]
    plain = K.plain_forward(toks, w, cfg).float()
    core = core_for(d, dtype, name)
    whole = stepwise(core, "a", toks, [300])
    single = stepwise(core, "b", toks, [])
    tol = atol_for(name, dtype, plain)
    keep = None if dtype == "float32" else well_conditioned(toks, w, cfg, plain, tol)
    record(f"Kudadra {name} {dtype} token by token", max(error(single, plain, dtype, keep), error(whole, plain, dtype, keep)),
           logits_std(plain))
    assert error(whole, plain, dtype, keep) <= tol and error(single, plain, dtype, keep) <= tol
    assert keep is None or keep.float().mean() > 0.95
    core.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["P", "Q", "R"])
def test_a_batch_of_unequal_requests_equals_each_alone_and_slots_are_used_again(tmp_path, name, dtype):
    d, cfg, w = make_model(tmp_path, name, dtype, seed=6)
    rng = random.Random(7)
    toks = {r: [rng.randrange(cfg["vocab"]) for _ in range(n)] for r, n in (("a", 75), ("b", 140), ("c", 9), ("d", 33), ("e", 52))}
    core = core_for(d, dtype, name, max_seqs=3)
    alone = {r: stepwise(core, r, t, [len(t) - 3]) for r, t in toks.items()}
    # together: a decodes while b and c bring portions; c ends and d takes its slot in the next step; then e takes a's
    got = {r: [] for r in toks}

    def step(*feeds, end=()):
        entries = []
        for r, c in feeds:
            if not core.is_open(r):
                core.open(r)
            at = sum(x.shape[0] for x in got[r])
            entries.append(StepEntry(r, toks[r][at:at + c], list(range(c))))
        out = core.step(entries).float().cpu()
        at = 0
        for r, c in feeds:
            got[r].append(out[at:at + c])
            at += c
        for r in end:
            core.close(r)

    step(("a", 70))
    step(("a", 1), ("b", 100), ("c", 7))
    step(("c", 2), ("a", 1), ("b", 2), end=["c"])
    step(("b", 37), ("d", 33), ("a", 1), end=["d"])
    step(("a", 1), ("b", 1))
    step(("a", 1), end=["a", "b"])
    step(("e", 50))
    step(("e", 2), end=["e"])
    core.cache.check()
    assert core.cache.free_slots == 3
    plain = {r: K.plain_forward(t, w, cfg).float() for r, t in toks.items()}
    tol = atol_for(name, dtype, plain)
    worst = 0.0
    for r in toks:
        both = torch.cat(got[r])
        keep = None if dtype == "float32" else well_conditioned(toks[r], w, cfg, plain[r], tol)
        worst = max(worst, error(both, plain[r], dtype, keep))
        assert error(both, plain[r], dtype, keep) <= tol, r
        # the batch and the request alone run the same kernels on the same numbers, up to the order of split sums
        assert error(both, alone[r], dtype) <= (2e-5 if dtype == "float32" else tol), r
    record(f"Kudadra {name} {dtype} batch", worst, logits_std(plain))
    core.runner.check_device_errors()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["P", "Q", "R"])
def test_greedy_generation_through_the_entry_point(tmp_path, name, dtype):
    d, cfg, w = make_model(tmp_path, name, dtype, seed=10)
    rng = random.Random(1)
    prompts = [[rng.randrange(cfg["vocab"]) for _ in range(n)] for n in (1, 9, 70, 23, 41)]
    eng = Engine(d, dtype=dtype, max_seq_len=160, max_batch_tokens=48, page_size=PAGE_SIZE[name], num_pages=40,
                 max_seqs=3, chunk_size=16)
    outs, why = eng.generate(prompts, max_new_tokens=12, temperature=0.0, eos_token_id=-1, return_reasons=True)
    assert why == ["length"] * 5 and all(len(o) == 12 for o in outs)
    margin_rel = 3e-4 if dtype == "float32" else 3.0 * KUDADRA_BF16_WORST_REL[name]
    for p, o in zip(prompts, outs):
        seq = list(p)
        for tok in o:
            lg = K.plain_forward(seq, w, cfg)[-1].float()
            top = torch.topk(lg, 2).values
            assert tok == int(torch.argmax(lg)) or float(top[0] - top[1]) < margin_rel * float(lg.std()), (seq, tok)
            seq.append(tok)
    eng.core.cache.check()
    assert eng.core.cache.free_slots == 3
    eng.core.runner.check_device_errors()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("M", [1, 7, 40, 130, 700])
def test_gated_activation_in_the_contractions_epilogue(dtype, M):
    """Every contraction kernel's GLU epilogue with the clamped gate (few rows: the decode kernel, split along K or not;
    up to 128 rows and beyond: the two tcgen05 kernels; float32: the CUDA-core kernel) against the contraction followed
    by the activation kernel, and against the formula."""
    from lightllm_b200.parts import linear as L
    torch.manual_seed(M)
    for K_, I in ((64, 48), (896, 1216), (136, 100)):
        x = (torch.randn(M, K_) * 0.7).to(DT[dtype])
        w = (torch.randn(2 * I, K_) / K_ ** 0.5 * 2).to(DT[dtype])
        pre = x.double() @ w.double().T
        g, u = pre[:, 0::2].clamp(max=1.25), pre[:, 1::2].clamp(-1.25, 1.25)
        want = g * torch.sigmoid(1.702 * g) * (u + 1.0)
        args = (dev(x), dev(w), None, ops.GLU_CLAMPED_SWISH, 1.702, 1.25, 1.0)
        fused = L.linear_glu(*args)
        L.FUSE_GLU = False
        try:
            apart = L.linear_glu(*args)
        finally:
            L.FUSE_GLU = True
        close(fused, want, dtype, f"fused clamped gate {M}x{K_}x{I}", rel=None if dtype == "float32" else 1e-2)
        close(apart, want, dtype, f"clamped gate behind the contraction {M}x{K_}x{I}", rel=None if dtype == "float32" else 1.5e-2)


def test_command_lines_serve_the_design(tmp_path):
    """``random_model`` writes a folder from a config.json of the design; ``generate`` continues a prompt greedily as the
    plain implementation does and samples the same tokens for the same seed; ``bench_server`` runs its users."""
    import json
    import re
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

    def run_cli(module, *args):
        env = dict(os.environ, PYTHONPATH=root + os.pathsep + os.environ.get("PYTHONPATH", ""))
        proc = subprocess.run([sys.executable, "-m", module, *map(str, args)], stdout=subprocess.PIPE, stderr=subprocess.PIPE,
                              text=True, env=env, timeout=600, cwd=root)
        assert proc.returncode == 0, proc.stderr[-3000:]
        return proc.stdout

    cfg = config("P")
    cfg_path = str(tmp_path / "config.json")
    with open(cfg_path, "w") as f:
        json.dump(cfg, f)
    d = str(tmp_path / "model")
    run_cli("lightllm_b200.cli.random_model", cfg_path, d, 4, "--store-dtype", "float32")
    from tests.plain.qwen2_plain import read_safetensors
    w = {k: v.double() for k, v in read_safetensors(os.path.join(d, "model.safetensors")).items()}
    prompt = [5, 17, 3, 99, 250, 7]
    out = run_cli("lightllm_b200.cli.generate", d, *prompt, "--temperature", 0, "--max-new-tokens", 8, "--dtype", "float32",
                  "--max-seq-len", 64)
    got = [int(t) for t in re.search(r"generated:\s*([\d ]+)", out).group(1).split()]
    seq = list(prompt)
    for tok in got:
        lg = K.plain_forward(seq, w, cfg)[-1]
        top = torch.topk(lg, 2).values
        assert tok == int(torch.argmax(lg)) or float(top[0] - top[1]) < 1e-4, (seq, tok)
        seq.append(tok)
    assert len(got) == 8
    pick = lambda s: re.search(r"generated:\s*([\d ]+)", s).group(1)
    a = run_cli("lightllm_b200.cli.generate", d, 1, 2, 3, "--seed", 5, "--max-seq-len", 64)
    b = run_cli("lightllm_b200.cli.generate", d, 1, 2, 3, "--seed", 5, "--max-seq-len", 64)
    assert pick(a) == pick(b)
    out = run_cli("lightllm_b200.cli.bench_server", d, 128, 64)
    assert "Hidden dim=44" in out and "vocab=301" in out


@pytest.mark.parametrize("name", ["P", "Q"])
def test_weights_stored_in_32_bits_served_in_bfloat16(tmp_path, name):
    """A folder stored in float32 run with bfloat16 activations: tensors stored in 32 bits stay so (CUDA-core
    contractions with bfloat16 operands and float weights), the attention and recurrence kernels are the bfloat16 ones."""
    cfg = config(name)
    w = random_weights(cfg, 12, store=torch.float32)
    d = write_model(cfg, w, str(tmp_path / "model32"))
    wd = {k: v.double() for k, v in w.items()}
    rng = random.Random(5)
    toks = [rng.randrange(cfg["vocab"]) for _ in range(150)]
    plain = K.plain_forward(toks, wd, cfg).float()
    got = stepwise(core_for(d, "bfloat16", name), "a", toks, [70, 2, 33, 30])
    tol = atol_for(name, "bfloat16", plain)
    keep = well_conditioned(toks, wd, cfg, plain, tol)
    record(f"Kudadra {name} float32-stored bfloat16", error(got, plain, "bfloat16", keep), logits_std(plain))
    assert error(got, plain, "bfloat16", keep) <= tol and keep.float().mean() > 0.95
