"""Bulitar on the GPU: every new kernel alone against the plain functions, then the model through the engine's own step
function, cache manager, scheduler and replay tool against the plain implementation, on four tiny configurations."""
import math
import random

import numpy as np
import pytest
import torch

from lightllm_b200 import Engine, EngineCore, EngineOptions, StepEntry
from lightllm_b200.csrc import ops
from tests.bulitar_configs import CONFIGS, PAGE_SIZE, config, random_weights, write_model
from tests.plain import bulitar_plain as P
from tests.tolerances import BULITAR_BF16_WORST_REL, FLOAT32_ATOL, logits_std, record
from tests.trace_util import Trace, compare_with_plain, run_trace

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def dev(t, dtype=None):
    return t.to(DEV, dtype=dtype).contiguous()


def i32(xs):
    return dev(torch.tensor(list(xs), dtype=torch.int32))


def close(got, want, dtype, what, rel=None):
    """float32: 2e-5 of the result's scale; bfloat16: a few roundings of 2^-9."""
    scale = float(want.abs().max()) + 1e-6
    tol = (2e-5 if dtype == "float32" else 2.5e-2) * scale if rel is None else rel * scale
    err = float((got.double().cpu() - want.double()).abs().max())
    assert err <= tol, f"{what}: max |diff| {err:.3e} > {tol:.3e}"


def spans_of(parts):
    """Device arrays (span_row, span_len, span_pos, span_slot, count) for parts (request, slot, from, to)."""
    starts = np.cumsum([0] + [b - a for _, _, a, b in parts])[:-1]
    return (i32(starts), i32(b - a for _, _, a, b in parts), i32(a for _, _, a, _ in parts), i32(s for _, s, _, _ in parts),
            len(parts))


# ---------------------------------------------------------------------------------------------------------------------
# kernels alone
# ---------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("D", [44, 320, 1500, 5000])
@pytest.mark.parametrize("wdtype", ["float32", "bfloat16"])
def test_layer_norm_without_bias(D, wdtype):
    torch.manual_seed(D)
    x = torch.randn(11, D) * 3 + 1.5
    w = (1 + 0.1 * torch.randn(D)).to(DT[wdtype])
    want = P.layer_norm(x.double(), w.double(), 1e-5)
    out = torch.empty(11, D, device=DEV)
    ops.layernorm(dev(x), dev(w), None, 1e-5, out)
    close(out, want, "float32", "layer norm")
    rows = torch.tensor([10, 0, 5], dtype=torch.int32)
    out = torch.empty(3, D, device=DEV, dtype=DT[wdtype])
    ops.layernorm(dev(x), dev(w), None, 1e-5, out, rows=dev(rows))
    close(out, want[rows.long()], wdtype, "layer norm of rows")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embedding_scaled_and_kept(dtype):
    torch.manual_seed(1)
    table = torch.randn(50, 36).to(DT[dtype])
    ids = torch.tensor([3, 49, 0, 3], dtype=torch.int32)
    out = torch.empty(4, 36, device=DEV)
    copy = torch.empty(4, 36, device=DEV, dtype=DT[dtype])
    ops.embedding(dev(ids), dev(table), out, scale=12.0, copy=copy)
    want = table.float()[ids.long()] * 12.0
    assert torch.equal(out.cpu(), want) and torch.equal(copy.cpu(), want.to(DT[dtype]))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("taps", [1, 2, 3, 4])
def test_short_convolution_with_rotation_and_head_norms(dtype, taps):
    """Three requests over three launches: spans that begin a request, continue one (from the tail another launch left,
    also when the span is shorter than the tail) and single tokens; a slot that a finished request used is taken
    again.  q: rotated with scaled frequencies, unit root mean square; k: the same into cache rows; v: SiLU, unit
    length, scaled, of another head size."""
    torch.manual_seed(taps)
    H, G, hd, vd, rot = 3, 2, 12, 7, 8
    C, extra = (H + G) * hd + G * vd, 5
    lens = {"a": 23, "b": 14, "c": 9}
    proj = {r: torch.randn(n, C + extra).to(DT[dtype]) for r, n in lens.items()}
    w = torch.randn(C, taps)
    rot_cfg = {"dims": rot, "base": 300.0, "scaling": {"factor": 4.0, "original": 16, "fast": 4.0, "slow": 1.0}}
    freq, mag = P.rotary_frequencies(rot_cfg)
    want = {}
    for r, n in lens.items():
        y = P.short_conv(proj[r].double()[:, :C], w.double())
        pos = torch.arange(n)
        q = P.unit_rms(P.rotate_pairs(y[:, :H * hd].reshape(n, H, hd), pos, rot_cfg), 1e-5)
        k = P.unit_rms(P.rotate_pairs(y[:, H * hd:(H + G) * hd].reshape(n, G, hd), pos, rot_cfg), 1e-5)
        v = y[:, (H + G) * hd:].reshape(n, G, vd)
        v = v * torch.sigmoid(v)
        v = v / torch.sqrt((v * v).sum(-1, keepdim=True) + 1e-6) * 0.25
        want[r] = (q, k, v)
    state = torch.full((3, 4 + (taps - 1) * C), float("nan"), device=DEV)          # the tail lies 4 floats into a slot
    kc = torch.full((64, G, hd), float("nan"), device=DEV, dtype=DT[dtype])
    slot_of = {"a": 0, "b": 24, "c": 40}

    def run(parts):
        rows = dev(torch.cat([proj[r][a:b] for r, _, a, b in parts]))
        T = rows.shape[0]
        q = torch.empty(T, H * hd, device=DEV, dtype=DT[dtype])
        v = torch.empty(T, G * vd, device=DEV)
        slots = i32(slot_of[r] + p for r, _, a, b in parts for p in range(a, b))
        sp = spans_of(parts)
        segs = [ops.ConvSegment(0, H, hd, q, rotary_dim=rot, norm="rms", eps=1e-5),
                ops.ConvSegment(H * hd, G, hd, kc, to_cache=True, rotary_dim=rot, norm="rms", eps=1e-5),
                ops.ConvSegment((H + G) * hd, G, vd, v, act="silu", norm="unit", eps=1e-6, scale=0.25)]
        ops.conv_prepare(rows, 0, C, dev(w), segs, sp, state if taps > 1 else None, 4, slots, dev(freq.float()), mag)
        if taps > 1:
            ops.conv_tail_update(rows, 0, C, taps, sp, state, 4)
        at = 0
        for r, _, a, b in parts:
            n = b - a
            close(q[at:at + n].view(n, H, hd), want[r][0][a:b], dtype, f"q of {r}[{a}:{b}]")
            close(v[at:at + n].view(n, G, vd), want[r][2][a:b], "float32" if dtype == "float32" else dtype, f"v of {r}[{a}:{b}]")
            close(kc[slot_of[r] + a: slot_of[r] + b], want[r][1][a:b], dtype, f"k rows of {r}[{a}:{b}]")
            at += n

    run([("a", 0, 0, 10), ("c", 1, 0, 9)])                       # c ends here; its slot 1 is used again by b
    run([("a", 0, 10, 11), ("b", 1, 0, 1)])                      # single tokens: spans shorter than the tail
    run([("b", 1, 1, 2), ("a", 0, 11, 12)])
    run([("b", 1, 2, 14), ("a", 0, 12, 23)])
    if taps > 1:
        tail = state[0, 4:].view(taps - 1, C).cpu()
        assert torch.equal(tail, proj["a"][23 - (taps - 1):, :C].float())


@pytest.mark.parametrize("blocked", [False, True])
@pytest.mark.parametrize("H,G,d,e", [(3, 1, 12, 20), (2, 2, 24, 9), (4, 2, 64, 64), (2, 1, 128, 32), (1, 1, 256, 40), (2, 2, 16, 300)])
def test_delta_rule_kernel_over_spans_and_slots(H, G, d, e, blocked):
    """Three requests in one launch: one from its first token, one that continues from a state another launch left (in
    a slot that a finished request used before), one single token; the state lies behind other floats of its slot."""
    torch.manual_seed(d + e)
    lens = {"a": 37, "b": 21, "c": 18}
    mk = lambda n, w: torch.randn(n, w)
    data = {}
    for r, n in lens.items():
        q = torch.nn.functional.normalize(mk(n, G * d).view(n, G, d), dim=-1) * d ** -0.5
        k = torch.nn.functional.normalize(mk(n, G * d).view(n, G, d), dim=-1)
        g = torch.rand(n, H, d) * 0.5 + 0.5
        g[n // 2] = 1e-30                          # a token that forgets nearly everything, in every channel
        g[:, :, 0] = 1.0                           # a channel that never decays
        data[r] = dict(q=q, k=k, v=mk(n, H * e).view(n, H, e), g=g, b=mk(n, H + 3))
    want = {}
    for r, n in lens.items():
        x = {k_: v_.double() for k_, v_ in data[r].items()}
        beta = torch.sigmoid(x["b"][:, 1:1 + H])
        want[r] = torch.stack([P.delta_rule(x["q"][:, h // (H // G)], x["k"][:, h // (H // G)], x["v"][:, h], x["g"][:, h],
                                            beta[:, h]) for h in range(H)], dim=1)
    off = 5
    state = torch.full((4, off + H * d * e + 2), float("nan"), device=DEV)
    got = {}

    def run(parts):
        cat = lambda key: dev(torch.cat([data[r][key][a:b] for r, _, a, b in parts]))
        T = sum(b - a for _, _, a, b in parts)
        o = torch.empty(T, H * e, device=DEV)
        bsrc = cat("b")
        ops.delta_rule(cat("q").view(T, -1), cat("k").view(T, -1), cat("v").view(T, -1), torch.log(cat("g")).view(T, -1),
                       bsrc[:, 1:1 + H], spans_of(parts), H, G, d, e, state, off, o, blocked=blocked)
        at = 0
        for r, _, a, b in parts:
            got[(r, a, b)] = o[at:at + b - a].cpu()
            at += b - a

    run([("a", 2, 0, 17), ("c", 0, 0, 18)])
    run([("a", 2, 17, 18), ("b", 0, 0, 2)])
    run([("b", 0, 2, 21), ("a", 2, 18, 37)])
    for (r, a, b), o in got.items():
        close(o.view(b - a, H, e), want[r][a:b], "float32", f"delta rule {r}[{a}:{b}]", rel=3e-5)
    assert torch.isnan(state[2, :off]).all() and torch.isnan(state[2, off + H * d * e:]).all()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,R", [(9, 5), (37, 5), (3, 40), (50, 64), (16, 33), (17, 96)])
def test_second_half_of_a_low_rank_pair(dtype, T, R):
    """Few rows take a kernel with a warp an output, more rows one with sixteen rows a block."""
    torch.manual_seed(5 + T)
    off, H, per = 7, 3, 11
    x = torch.randn(T, off + R + 2).to(DT[dtype])
    w = torch.randn(H * per, R).to(DT[dtype])
    bias, rate = torch.randn(H * per), torch.rand(H) + 0.5
    z = x.double()[:, off:off + R] @ w.double().T
    for mode, want, out_dtype in ((None, z, dtype), ("sigmoid", torch.sigmoid(z + bias.double()), "float32"),
                                  ("log_decay", -rate.double().repeat_interleave(per) *
                                   torch.nn.functional.softplus(z + bias.double()), "float32")):
        out = torch.empty(T, H * per, device=DEV, dtype=DT[out_dtype])
        ops.low_rank_up(dev(x), off, dev(w), out, bias=None if mode is None else dev(bias), mode=mode,
                        rate=dev(rate) if mode == "log_decay" else None)
        close(out, want, out_dtype, f"low rank, mode {mode}", rel=None if out_dtype == "float32" else 8e-3)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("E,top", [(5, 2), (8, 3), (1, 1), (4, 4), (70, 6)])
def test_routing_and_expert_weights(dtype, E, top):
    """Scores, the choice with the correction, weights without it.  Where the plain scores of the last expert chosen and
    the first one left out lie closer than rounding can tell, either choice is right."""
    torch.manual_seed(E)
    T, D, F = 37, 44, 6
    x = torch.randn(T, D).to(DT[dtype])
    W = {"m.router": torch.randn(E, D) * 0.3, "m.correction": torch.randn(E) * 0.3}
    ids = torch.empty(T, top, dtype=torch.int32, device=DEV)
    wts = torch.empty(T, top, device=DEV)
    dense = torch.empty(T, E, device=DEV)
    ops.moe_route(dev(x), dev(W["m.router"]), dev(W["m.correction"]), top, 2.5, ids, wts, dense)
    s = torch.sigmoid(x.double() @ W["m.router"].double().T)
    choice = s + W["m.correction"].double()
    order = choice.sort(-1, descending=True)
    margin = (order.values[:, top - 1] - order.values[:, top]) if top < E else torch.full((T,), 1.0, dtype=torch.float64)
    sure = margin > 1e-4
    got_sets = [set(r) for r in ids.cpu().tolist()]
    for t in range(T):
        if sure[t]:
            assert got_sets[t] == set(order.indices[t, :top].tolist()), t
        assert ids.cpu()[t].tolist() == sorted(ids.cpu()[t].tolist(), key=lambda e_: -float(choice[t, e_]))      # in order
    close(wts, torch.gather(s, 1, ids.cpu().long()) * 2.5, "float32", "weights", rel=1e-5)
    want_dense = torch.zeros(T, E, dtype=torch.float64).scatter(1, ids.cpu().long(), torch.gather(s, 1, ids.cpu().long()) * 2.5)
    close(dense, want_dense, "float32", "dense weights", rel=1e-5)
    assert int((dense != 0).sum()) == T * top
    # softmax scores, renormalised
    ops.moe_route(dev(x), dev(W["m.router"]), None, top, 1.0, ids, wts, dense, softmax=True, renormalize=True)
    sm = torch.softmax(x.double() @ W["m.router"].double().T, -1)
    picked = torch.gather(sm, 1, ids.cpu().long())
    close(wts, picked / picked.sum(-1, keepdim=True), "float32", "softmax weights", rel=1e-5)
    # the activations of the experts a row did not choose become exact zeros, whatever they hold
    act = torch.randn(T, E * F).to(DT[dtype])
    act[0, 0] = float("inf")
    a = dev(act)
    ops.moe_route(dev(x), dev(W["m.router"]), dev(W["m.correction"]), top, 2.5, ids, wts, dense)
    ops.moe_scale(a, dense, E, F)
    want = act.double().view(T, E, F) * dense.cpu().double()[:, :, None]
    want[dense.cpu()[:, :, None].expand(T, E, F) == 0] = 0.0
    got = a.double().cpu().view(T, E, F)
    fin = torch.isfinite(want)
    assert torch.equal(torch.isfinite(got), fin)
    close(got[fin], want[fin], dtype, "scaled activations", rel=None if dtype == "float32" else 8e-3)


def paged(k, npages, page, dtype, seed=0):
    g = torch.Generator().manual_seed(seed)
    n = k.shape[0]
    pages = torch.randperm(npages, generator=g)[: -(-n // page)].to(torch.int32)
    cache = torch.full((npages * page, *k.shape[1:]), float("nan"), dtype=DT[dtype])
    cache[pages[torch.arange(n) // page].long() * page + torch.arange(n) % page] = k
    return dev(cache), dev(pages.view(1, -1))


def plain_rows(q, k, v, start, scale, chunk):
    """Attention of the rows at positions start.. over the keys 0..: the whole sequence through the plain function."""
    n = start + q.shape[0]
    full_q = torch.zeros(n, *q.shape[1:], dtype=torch.float64)
    full_q[start:] = q.double()
    return P.chunked_softmax_attention(full_q, k.double()[:n], v.double()[:n], scale, chunk)[start:]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("chunk", [1, 7, 50, 120])
def test_cuda_core_attention_with_chunks(dtype, chunk):
    """Portions that begin inside a chunk and cross one or several chunk borders, in tiles of rows and row by row with
    the keys in pieces, and single tokens at a chunk's first and last position; values narrower than keys."""
    torch.manual_seed(chunk)
    H, G, hd, vd, page, n = 6, 2, 24, 10, 8, 333
    k, v = torch.randn(n, G, hd).to(DT[dtype]), torch.randn(n, G, vd).to(DT[dtype])
    kc, bt = paged(k, 64, page, dtype)
    vc, _ = paged(v, 64, page, dtype)
    first = (n - 1) // chunk * chunk
    for start, rows, bq, nsplit in ((290, 43, 4, 1), (290, 43, 1, 3), (first, 1, 1, 1), (first - 1 if first else 0, 1, 1, 4),
                                    (0, 20, 16, 1), (n - 1, 1, 1, 2)):
        q = (torch.randn(rows, H, hd) * 1.5).to(DT[dtype])
        want = plain_rows(q, k, v, start, 0.3, chunk)
        out = torch.empty(rows, H * vd, device=DEV, dtype=DT[dtype])
        tq0 = list(range(0, rows, bq))
        scratch = torch.empty(ops.attention_scratch_floats(len(tq0), H, vd, bq, nsplit), device=DEV) if nsplit > 1 else None
        ops.paged_attention_simt(dev(q).view(rows, H * hd), kc, vc, out, i32([0] * len(tq0)), i32(tq0), len(tq0), i32([0]),
                                 i32([rows]), i32([start]), bt, bt.shape[1], page, H, G, hd, -chunk, 0.3, bq, nsplit, scratch,
                                 v_head_dim=vd)
        close(out.view(rows, H, vd), want, dtype, f"chunk {chunk}: start {start}, {rows} rows, bq {bq}, {nsplit} pieces",
              rel=None if dtype == "float32" else 1.5e-2)


@pytest.mark.parametrize("hd", [64, 128])
@pytest.mark.parametrize("chunk", [1, 5, 129, 200, 256])
def test_tensor_core_attention_with_chunks(hd, chunk):
    """The tcgen05 prefill kernel (whole key ranges and ranges cut into pieces) and the mma.sync decode kernel (pieces
    merged in a cluster and through scratch) under the chunk mask: tiles of rows that cross chunk borders, whole key
    tiles that some rows of a tile do not see, single tokens at a chunk's first position."""
    torch.manual_seed(hd + chunk)
    H, G, page, n = 4, 2, 16, 700
    k, v = torch.randn(n, G, hd).to(torch.bfloat16), torch.randn(n, G, hd).to(torch.bfloat16)
    kc, bt = paged(k, 64, page, "bfloat16")
    vc, _ = paged(v, 64, page, "bfloat16")
    scale = 1.5 / hd ** 0.5
    from lightllm_b200.engine.batch import Span, StepContext
    for start, rows, pieces in ((0, 300, None), (380, 320, 2), (690, 10, None), (250, 135, None)):
        q = torch.randn(rows, H, hd).to(torch.bfloat16)
        out = torch.empty(rows, H * hd, device=DEV, dtype=torch.bfloat16)
        ctx = StepContext()
        ctx.spans, ctx.device = [Span("a", 0, start, rows, 0)], DEV
        ctx.iota, ctx.zeros = i32([0]), i32([0])
        ts, tq, nt, cut = ctx.attention_items(1, -chunk, pieces, H, 296)
        ops.paged_attention_tcgen05(dev(q).view(rows, H * hd), kc, vc, out, ts, tq, nt, i32([0]), i32([rows]), i32([start]),
                                    bt, bt.shape[1], page, H, G, hd, -chunk, scale, cut=cut)
        ops.check_async_errors(DEV)
        close(out.view(rows, H, hd), plain_rows(q, k, v, start, scale, chunk), "bfloat16",
              f"tcgen05, chunk {chunk}, start {start}, {rows} rows, pieces of {pieces}", rel=1.5e-2)
    for pos in (n - 1, (n - 1) // chunk * chunk, max(0, (n - 1) // chunk * chunk - 1)):
        for nsplit in (1, 4, 20):
            q = torch.randn(1, H, hd).to(torch.bfloat16)
            out = torch.empty(1, H * hd, device=DEV, dtype=torch.bfloat16)
            scratch = None
            if nsplit > ops.decode_mma_cluster_splits():
                scratch = torch.empty(ops.attention_scratch_floats(1, H, hd, 1, nsplit), device=DEV)
            ops.paged_decode_mma(dev(q).view(1, H * hd), kc, vc, out, i32([0]), i32([0]), 1, i32([0]), i32([pos]), bt,
                                 bt.shape[1], page, H, G, hd, -chunk, scale, nsplit, scratch)
            close(out.view(1, H, hd), plain_rows(q, k, v, pos, scale, chunk), "bfloat16",
                  f"decode at {pos}, chunk {chunk}, {nsplit} pieces", rel=1.5e-2)


# ---------------------------------------------------------------------------------------------------------------------
# the model through the engine
# ---------------------------------------------------------------------------------------------------------------------
def variant_config(name, dtype, sharp=1.0):
    """The configuration a test runs.  In bfloat16 every expert is chosen (top = experts): which expert a token takes is
    a discrete choice that rounding flips when two scores lie close, and a flipped expert is not an error of the engine.
    The choice itself is tested on the kernel (where close calls are told apart) and, through the model, in float32."""
    cfg = config(name)
    for layer in cfg["layers"]:
        if dtype == "bfloat16" and layer.get("mlp") is not None:
            layer["mlp"]["router"]["top"] = layer["mlp"]["router"]["experts"]
        if layer["type"] == "attention":
            layer["mixer"]["scale"] *= sharp
    return cfg


def make_model(tmp_path, name, dtype, seed=3, sharp=1.0):
    cfg = variant_config(name, dtype, sharp)
    w = random_weights(cfg, seed, store=DT[dtype])
    d = write_model(cfg, w, str(tmp_path / f"bul_{name}_{seed}_{dtype}"))
    return d, cfg, {k: v.double() for k, v in w.items()}


def core_for(d, dtype, name, pages=64, max_seqs=4, max_tokens=1024, graphs=True):
    return EngineCore(d, EngineOptions(dtype=dtype, max_seq_len=max_tokens, max_batch_tokens=max_tokens,
                                       page_size=PAGE_SIZE[name], num_pages=pages, max_seqs=max_seqs,
                                       use_cuda_graphs=graphs))


def plain_logits(toks, w, cfg):
    return P.forward(toks, cfg, w)[0].float()


def atol_for(name, dtype, plain):
    """float32: the largest difference of any logit, 1e-4 on logits of order one.  bfloat16: the root mean square over a
    row of logits (mean taken off), at most twice the worst that a recorded run showed, relative to the logits' spread."""
    std = logits_std(plain)
    return (FLOAT32_ATOL * max(1.0, std)) if dtype == "float32" else 2.0 * BULITAR_BF16_WORST_REL[name] * std


def row_errors(got, plain, dtype):
    d = (got.double() - plain.double())
    if dtype == "float32":
        return d.abs().max(-1).values
    return (d - d.mean(-1, keepdim=True)).pow(2).mean(-1).sqrt()


def error(got, plain, dtype) -> float:
    return float(row_errors(got, plain, dtype).max())


LENGTHS = {"U": [1, 2, 17, 33, 70, 150, 64, 49], "V": [3, 40, 131, 330, 129, 520, 64, 257], "W": [1, 5, 40, 90, 33, 64, 17, 200],
           "X": [1, 3, 20, 45, 16, 70, 33, 9]}


def build_trace(name, cfg, seed=11):
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
    tr.mixed([f"m{rid}" for rid in seqs], prompt_len, seed=5, sizes=(2, 3, 7, 16, 40, 130) if name == "V" else (2, 3, 5, 7, 16))
    return tr, seqs


@pytest.mark.parametrize("name", sorted(CONFIGS))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_all_regimes(name, dtype, tmp_path):
    """Through bin/trace_run: whole prompts, the last tokens one by one, portions down to two tokens, and up to four
    live requests mixed in a pool so small that pages and state slots are used again."""
    d, cfg, w = make_model(tmp_path, name, dtype)
    tr, seqs = build_trace(name, cfg)
    once = {rid: plain_logits(toks, w, cfg) for rid, toks in seqs.items()}
    plain = {f"{regime}{rid}": lg for rid, lg in once.items() for regime in "wtpm"}
    got = run_trace(d, dtype, tr, str(tmp_path / "out"), ["--page-size", str(PAGE_SIZE[name])])
    worst = compare_with_plain(tr, got, plain, atol_for(name, dtype, once), f"Bulitar {name} {dtype}", rms=dtype != "float32")
    record(f"replay Bulitar {name} {dtype} ({len(tr.steps)} steps, pool for {tr.max_tokens} tokens)", worst, logits_std(once))


def stepwise(core, rid, toks, cuts):
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
@pytest.mark.parametrize("name", ["U", "V", "W"])
def test_sharp_attention_sees_far_keys_and_chunk_edges(tmp_path, name, dtype):
    """The attention's scale multiplied by 6, so that single keys carry a row's attention: a key that is lost (far back,
    at a page's border, the first of a chunk) or seen though it lies in the chunk before moves the logits by far more
    than rounding.  Prompt in portions that end inside pages and chunks, then 60 tokens one by one, so that chunk
    borders pass under decoded tokens.  W has a layer without a mask: its last rows look hundreds of keys back."""
    d, cfg, w = make_model(tmp_path, name, dtype, seed=8, sharp=6.0)
    rng = random.Random(2)
    n = 420 if name == "V" else 200
    toks = [rng.randrange(cfg["vocab"]) for _ in range(n)]
    plain = plain_logits(toks, w, cfg)
    core = core_for(d, dtype, name)
    got = stepwise(core, "a", toks, [129, 2, 150 - 131, 31, 2, 64] if name == "V" else [9, 2, 16, 38, 2, 70])
    err = error(got, plain, dtype)
    record(f"sharp Bulitar {name} {dtype}", err, logits_std(plain))
    assert err <= atol_for(name + " sharp", dtype, plain)
    core.runner.check_device_errors()
    # the plain implementation itself shows what a chunk that is one position off would cost here
    for shift in (1, -1):
        cfg2 = variant_config(name, dtype, 6.0)
        edited = False
        for layer in cfg2["layers"]:
            mask = layer["mixer"].get("mask")
            if layer["type"] == "attention" and mask and mask["size"] + shift > 0:
                mask["size"] += shift
                edited = True
        if edited:
            off = error(plain_logits(toks, w, cfg2), plain, dtype)
            print(f"chunks off by {shift}: {off:.3e}; allowed: {atol_for(name + ' sharp', dtype, plain):.3e}")
            assert off > 1.5 * atol_for(name + " sharp", dtype, plain), (shift, off)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["U", "X"])
def test_prefill_equals_token_by_token_and_long_decoding(tmp_path, name, dtype):
    """A whole prompt in one step against the same tokens one by one from the first (300 single steps: the recurrent
    state and the convolutions' tails are carried through every one, chunk borders pass under decoded tokens only)."""
    d, cfg, w = make_model(tmp_path, name, dtype, seed=5)
    rng = random.Random(4)
    toks = [rng.randrange(cfg["vocab"]) for _ in range(300)]
    plain = plain_logits(toks, w, cfg)
    core = core_for(d, dtype, name)
    whole = stepwise(core, "a", toks, [300])
    single = stepwise(core, "b", toks, [])
    tol = atol_for(name, dtype, plain)
    record(f"Bulitar {name} {dtype} token by token", max(error(single, plain, dtype), error(whole, plain, dtype)), logits_std(plain))
    assert error(whole, plain, dtype) <= tol and error(single, plain, dtype) <= tol
    core.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["U", "V", "W"])
def test_a_batch_of_unequal_requests_equals_each_alone_and_slots_are_used_again(tmp_path, name, dtype):
    d, cfg, w = make_model(tmp_path, name, dtype, seed=6)
    rng = random.Random(7)
    toks = {r: [rng.randrange(cfg["vocab"]) for _ in range(n)] for r, n in (("a", 75), ("b", 140), ("c", 9), ("d", 33), ("e", 52))}
    core = core_for(d, dtype, name, max_seqs=3)
    alone = {r: stepwise(core, r, t, [len(t) - 3]) for r, t in toks.items()}
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

    # a decodes while b and c bring portions; c ends and d takes its slot in the next step; then e takes a's
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
    plain = {r: plain_logits(t, w, cfg) for r, t in toks.items()}
    tol = atol_for(name, dtype, plain)
    worst = 0.0
    for r in toks:
        both = torch.cat(got[r])
        worst = max(worst, error(both, plain[r], dtype))
        assert error(both, plain[r], dtype) <= tol, r
        # the batch and the request alone run the same kernels on the same numbers, up to the order of split sums
        assert error(both, alone[r], dtype) <= (2e-5 * max(1.0, logits_std(plain)) if dtype == "float32" else tol), r
    record(f"Bulitar {name} {dtype} batch", worst, logits_std(plain))
    core.runner.check_device_errors()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["U", "V", "W"])
def test_greedy_generation_through_the_entry_point(tmp_path, name, dtype):
    d, cfg, w = make_model(tmp_path, name, dtype, seed=10)
    rng = random.Random(1)
    prompts = [[rng.randrange(cfg["vocab"]) for _ in range(n)] for n in (1, 9, 70, 23, 41)]
    eng = Engine(d, dtype=dtype, max_seq_len=160, max_batch_tokens=48, page_size=PAGE_SIZE[name], num_pages=40,
                 max_seqs=3, chunk_size=16)
    outs, why = eng.generate(prompts, max_new_tokens=12, temperature=0.0, eos_token_id=-1, return_reasons=True)
    assert why == ["length"] * 5 and all(len(o) == 12 for o in outs)
    margin_rel = 3e-4 if dtype == "float32" else 3.0 * BULITAR_BF16_WORST_REL[name]
    for p, o in zip(prompts, outs):
        seq = list(p)
        for tok in o:
            lg = plain_logits(seq, w, cfg)[-1]
            top = torch.topk(lg, 2).values
            assert tok == int(torch.argmax(lg)) or float(top[0] - top[1]) < margin_rel * float(lg.std()), (seq, tok)
            seq.append(tok)
    eng.core.cache.check()
    assert eng.core.cache.free_slots == 3
    eng.core.runner.check_device_errors()


@pytest.mark.parametrize("T,E,top,D,F", [(300, 8, 2, 64, 48), (1000, 5, 1, 128, 2056), (257, 16, 3, 96, 136), (1, 8, 2, 64, 48),
                                         (3, 8, 2, 896, 2432), (5, 16, 3, 96, 136), (60, 8, 2, 64, 48)])
def test_grouped_experts_equal_every_expert_on_every_row(T, E, top, D, F):
    """The routed feed-forward on the grouped contractions (pairs sorted by expert, experts padded to whole tiles) and,
    for fewer pairs than experts, pair by pair, against the plain sum over the chosen experts and against the same part
    with every expert on every row; an expert that no row chose and experts with more rows than a tile are among them."""
    from lightllm_b200.parts.moe import RoutedExperts
    if not ops.has_tcgen05():
        pytest.skip("needs the tcgen05 contraction")
    torch.manual_seed(T + E)
    part = RoutedExperts("m", D, F, E, top, route_scale=2.5, correction=True, expert_prefix="e", weight_suffix="",
                         names={"gate": "gate", "up": "up", "down": "down"})
    W = {s.name: (torch.randn(s.shape) / (s.shape[-1] ** 0.5 if len(s.shape) == 2 else 1.0)).to(torch.bfloat16)
         for s in part.weight_specs()}
    W["m.correction"] = torch.randn(E).to(torch.bfloat16)
    W["m.correction"][E - 1] = -50.0                      # the last expert is never chosen
    part.bind({k: dev(v) for k, v in W.items()}, torch.bfloat16, DEV)
    x = torch.randn(T, D).to(torch.bfloat16)
    assert part.grouped_pays(T) or T * top < E
    grouped, dense = torch.zeros(T, D, device=DEV), torch.zeros(T, D, device=DEV)
    part.forward(dev(x), grouped)
    ops.check_async_errors(DEV)
    RoutedExperts.GROUPED = False
    try:
        part.forward(dev(x), dense)
    finally:
        RoutedExperts.GROUPED = True
    Wd = {k: v.double() for k, v in W.items()}
    want = P.moe(x.double(), Wd, "m", {"router": {"top": top, "scale": 2.5}})
    # rows whose choice hangs on a close call are judged against the engine's own other path only
    s = torch.sigmoid(x.double() @ Wd["m.router"].T) + Wd["m.correction"]
    order = s.sort(-1, descending=True).values
    sure = (order[:, top - 1] - order[:, top]) > 1e-3
    assert sure.float().mean() > 0.9 or T < 10
    close(grouped[sure.to(DEV)], want[sure], "bfloat16", "grouped experts against the plain sum", rel=2e-2)
    close(grouped, dense.double().cpu(), "bfloat16", "grouped experts against every expert on every row", rel=2e-2)


@pytest.mark.parametrize("name", ["V", "X"])
def test_chosen_experts_through_the_engine_in_bfloat16(tmp_path, name):
    """The bfloat16 engine with fewer experts chosen than there are: single tokens take the experts pair by pair, portions
    of 48 rows or more the grouped contractions (V; X's widths keep every expert on every row), the rest every expert on
    every row.  So that rounding cannot flip a choice, the corrections lie 2 apart (the same experts win for every token;
    their weights still follow the token's scores)."""
    cfg = config(name)
    w = random_weights(cfg, 12, store=torch.bfloat16)
    for k in w:
        if k.endswith("correction"):
            w[k] = (-2.0 * torch.arange(w[k].numel(), dtype=torch.float32)).to(torch.bfloat16)
    d = write_model(cfg, w, str(tmp_path / f"bul_{name}_experts"))
    wd = {k: v.double() for k, v in w.items()}
    rng = random.Random(9)
    toks = [rng.randrange(cfg["vocab"]) for _ in range(150)]
    plain = plain_logits(toks, wd, cfg)
    core = core_for(d, "bfloat16", name)
    got = stepwise(core, "a", toks, [100, 20, 2, 7])          # grouped, every expert on every row, then pair by pair
    err = error(got, plain, "bfloat16")
    record(f"Bulitar {name} bfloat16 chosen experts", err, logits_std(plain))
    assert err <= atol_for(name, "bfloat16", plain)
    core.runner.check_device_errors()


def test_command_lines_serve_the_design(tmp_path):
    """``random_model`` writes a folder from a config.json of the design (the ranks of the low-rank pairs given in it);
    ``generate`` continues a prompt greedily as the plain implementation does and samples the same tokens for the same
    seed; ``bench_server`` runs its users."""
    import json
    import os
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

    cfg = config("U")
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
        lg = P.forward(seq, cfg, w)[0][-1]
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
