"""Prefill and decode throughput of the Zisevik design (latent attention with a window and a sink,
retention, dense and routed feed-forwards between pre-norms over a 32-bit stream, a looped stack)
at layer sizes that resemble a real model's, beside the engine's closest other model (the hybrid
design Bavutar: attention and recurrent mixers over a 32-bit stream) at equal width and number of
layer visits, and each of the design's own kernels alone against its roofline, with the like
kernel of the closest model beside it.

    python -m sparseengine_b200.cli.zisevik_bench [--sizes 2048,4096] [--steps 20] [--warmup 3]

Random weights, bfloat16, one GPU, device-timed with CUDA events; inputs differ from step to step
and the weights of a step exceed the L2 cache.  ``bench.py --design zisevik`` prints the same
record as its one JSON line.
"""
from __future__ import annotations

import argparse
import json
import sys

import torch

from .hybrid_bench import PAGE_SIZE, VOCAB, _parts, _throughput, hybrid_config
from .kernel_bench import peaks, timed

WINDOW = 1024


def zisevik_config(width: int) -> dict:
    """Four layers, the two in the middle run three times (eight visits: five latent attention,
    three retention; six dense and two routed feed-forwards).  Latent attention: heads of 64 + 64
    (rotated) query/key dims, values of 64, a cached row of 192 + 64, a window of 1,024; retention:
    heads with a 128 x 128 state; feed-forwards: dense of 4 x width, or 8 experts of width each, 2 per
    token."""
    heads = width // 128
    lat = {"heads": 2 * heads, "dim": 64, "rot_dim": 64, "vdim": 64, "q_rank": width // 2, "kv_rank": 192,
           "mask": {"size": WINDOW}, "rot": {"base": 500000.0, "dims": 64}, "scale": 128 ** -0.5}
    ret = {"heads": heads, "dim": 128, "vdim": 128, "rot": {"base": 1e6, "dims": 128},
           "decay": [1.0 - 2.0 ** (-5 - 7 * i / max(1, heads - 1)) for i in range(heads)]}
    dense = {"kind": "dense", "ff": 4 * width}
    moe = {"kind": "moe", "expert": {"ff": width}, "router": {"experts": 8, "top": 2}}
    layers = [{"type": "latent_attention", "mixer": dict(lat), "mlp": moe}, {"type": "retention", "mixer": ret, "mlp": dense},
              {"type": "latent_attention", "mixer": dict(lat), "mlp": dense}, {"type": "latent_attention", "mixer": dict(lat), "mlp": moe}]
    return {"architecture": "Zisevik", "vocab": VOCAB, "width": width, "layers": layers, "loop": {"start": 1, "stop": 3, "times": 3},
            "norm": {"eps": 1e-6}, "max_position": 16384}


def _kernels(width: int, cases, pk: dict) -> dict:
    """Each kernel of the design alone: microseconds, the bytes it has to move (inputs read once,
    outputs written once) or the operations it has to do, and the share of the measured copy
    bandwidth or bfloat16 matrix throughput that is; ``like: ...`` are kernels of the closest model
    on inputs of the same size.  ``cases``: (tokens, requests, keys each request already holds)."""
    from types import SimpleNamespace

    from ..csrc import ops
    dev = torch.device("cuda:0")
    cfg = zisevik_config(width)
    lat, ret = cfg["layers"][0]["mixer"], cfg["layers"][1]["mixer"]
    bf = torch.bfloat16
    out = {}
    for tokens, entries, held in cases:
        per = tokens // entries
        step = SimpleNamespace(token_seq=torch.arange(tokens, device=dev, dtype=torch.int32) // per,
                               cu_q=torch.arange(entries + 1, device=dev, dtype=torch.int32) * per,
                               seq_rows=torch.arange(entries, device=dev, dtype=torch.int32), num_seqs=entries, max_q_len=per,
                               positions=(torch.arange(tokens, device=dev, dtype=torch.int32) % per) + held)
        kv_len = torch.full((entries,), held + per, device=dev, dtype=torch.int32)
        rec = {}

        def add(name, fn, nbytes=None, flops=None, iters=20):
            ms = timed(fn, iters)
            r = {"us": round(ms * 1e3, 2)}
            if nbytes is not None:
                r.update(mbytes=round(nbytes / 1e6, 2), of_hbm_measured=round(nbytes / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 3))
            if flops is not None:
                r.update(gflop=round(flops / 1e9, 2), of_bf16_measured=round(flops / (ms * 1e-3) / 1e12 / pk["bf16_tflops"], 3))
            rec[name] = r

        # norm over the stream
        x32 = torch.randn(tokens, width, device=dev)
        y = torch.randn(tokens, width, device=dev, dtype=bf)
        w = torch.ones(width, device=dev, dtype=bf)
        o32, oa = torch.empty_like(x32), torch.empty_like(y)
        add("add_rmsnorm_stream", lambda: ops.add_rmsnorm_stream(x32, y, w, 1e-6, out32=x32, out_act=oa), tokens * width * 12)
        add("like: add_layernorm", lambda: ops.add_layernorm(x32, y, 2.0, w, w, 1e-6, out32=o32, out_act=oa), tokens * width * 12)
        # latent attention
        H, d, r, rank, qr = lat["heads"], lat["dim"], lat["rot_dim"], lat["kv_rank"], lat["q_rank"]
        D = rank + r
        pages = -(-(held + per) // PAGE_SIZE)
        table = torch.arange(entries * pages, device=dev, dtype=torch.int32).view(entries, pages)
        cache = (torch.randn(entries * pages, PAGE_SIZE, D, device=dev) * 0.5).to(bf)
        proj = torch.randn(tokens, qr + D, device=dev, dtype=bf)
        qw, kw = torch.ones(qr, device=dev, dtype=bf), torch.ones(rank, device=dev, dtype=bf)
        inv = (500000.0 ** (-torch.arange(0, r, 2, dtype=torch.float32) / r)).to(dev)
        cq = torch.empty(tokens, qr, device=dev, dtype=bf)
        add("latent_prep", lambda: ops.latent_prep(proj, qw, kw, inv, step.positions, step.token_seq, step.seq_rows, table, cache, cq,
                                                   q_rank=qr, rank=rank, rot=r, rotary_dim=r, eps=1e-6, page_size=PAGE_SIZE),
            tokens * (qr + D) * 4)
        q = torch.randn(tokens, H * (d + r), device=dev, dtype=bf)
        q_lat = torch.randn(H, tokens, rank, device=dev)
        qfull = torch.empty(tokens, H, D, device=dev, dtype=bf)
        add("latent_q_pack", lambda: ops.latent_q_pack(q_lat, q, inv, step.positions, qfull, heads=H, head_dim=d, rank=rank, rot=r,
                                                       rotary_dim=r), tokens * H * (rank * 4 + r * 2 + D * 2))
        sink = torch.zeros(H, device=dev)
        o_lat = torch.empty(tokens, H, rank, device=dev, dtype=bf)
        # keys a query sees: min(window, position + 1)
        seen = sum(min(WINDOW, held + i + 1) for i in range(per)) * entries
        key_rows = entries * min(held + per, WINDOW + per - 1)
        add("latent_attention_tiled", lambda: ops.latent_attention_tiled(
            qfull, cache, table, step.seq_rows, step.cu_q, kv_len, sink, o_lat, entries=entries, max_q_len=per, heads=H, rank=rank,
            rot=r, page_size=PAGE_SIZE, scale=0.09, window=WINDOW, max_keys=min(held + per, WINDOW + per - 1)),
            nbytes=key_rows * D * 2 + tokens * H * (D + rank) * 2, flops=2.0 * seen * H * (D + rank))
        if tokens <= 256:
            add("latent_attention_plain", lambda: ops.latent_attention_plain(
                q_lat, q, inv, cache, table, step.seq_rows, step.token_seq, step.positions, sink, o_lat, heads=H, head_dim=d,
                rank=rank, rot=r, rotary_dim=r, page_size=PAGE_SIZE, scale=0.09, window=WINDOW),
                nbytes=key_rows * D * 2 + tokens * H * (D + rank) * 2)
        # like: grouped-query attention of the closest model (head size 128, 4 query heads per key/value head, all keys)
        hq, hkv = width // 128, max(1, width // 512)
        cache2 = (torch.randn(entries * pages, 2, hkv, PAGE_SIZE, 128, device=dev) * 0.5).to(bf)
        q2, o2 = torch.randn(tokens, hq * 128, device=dev, dtype=bf), torch.empty(tokens, hq * 128, device=dev, dtype=bf)
        seen2 = sum(held + i + 1 for i in range(per)) * entries
        if per > 1:
            add("like: attn_prefill_tc (head size 128, all keys)", lambda: ops.attn_prefill_tc(
                q2, cache2, table, step.seq_rows, step.cu_q, kv_len, o2, entries=entries, max_q_len=per, num_heads=hq,
                num_kv_heads=hkv, head_dim=128, page_size=PAGE_SIZE, scale=0.09), flops=4.0 * seen2 * hq * 128)
        else:
            add("like: attn_decode (head size 128, all keys)", lambda: ops.attn_decode(
                q2, cache2, table, step.seq_rows, step.token_seq, step.positions, o2, num_heads=hq, num_kv_heads=hkv, head_dim=128,
                page_size=PAGE_SIZE, scale=0.09, max_keys=held + 1), nbytes=entries * (held + 1) * hkv * 128 * 4)
        # retention
        Hr, dr, dvr = ret["heads"], ret["dim"], ret["vdim"]
        qk, vv = Hr * dr, Hr * dvr
        proj_r = torch.randn(tokens, 2 * qk + 2 * vv, device=dev, dtype=bf) * 0.3
        inv_r = (1e6 ** (-torch.arange(0, dr, 2, dtype=torch.float32) / dr)).to(dev)
        q32, k32 = torch.empty(tokens, qk, device=dev), torch.empty(tokens, qk, device=dev)
        add("retention_prep", lambda: ops.retention_prep(proj_r, 0, qk, inv_r, step.positions, q32, k32, heads=Hr, head_dim=dr,
                                                         rotary_dim=dr, k_scale=dr ** -0.5), tokens * qk * 12)
        decay = torch.tensor(ret["decay"], device=dev, dtype=torch.float32)
        state = torch.zeros(entries, Hr * dr * dvr, device=dev)
        o_r = torch.empty(tokens, vv, device=dev)
        add("retention_scan", lambda: ops.retention_scan(q32, k32, proj_r, 2 * qk, decay, state, step, o_r, heads=Hr, head_dim=dr,
                                                         v_head_dim=dvr), tokens * (2 * qk * 4 + vv * 6) + entries * Hr * dr * dvr * 8, iters=5)
        rec["retention_scan"]["us_per_token_of_a_request"] = round(rec["retention_scan"]["us"] / per, 3)
        if per >= 16:
            # 32-bit FMAs of the closed form: scores (half of the 64 x 64 square is used), their product with the
            # values, the old state's part and the new state
            fma = tokens * Hr * (64 * dr * ((dvr + 31) // 32) + 64 * dvr + 2 * dr * dvr)
            add("retention_chunk", lambda: ops.retention_chunk(q32, k32, proj_r, 2 * qk, decay, state, step, o_r, heads=Hr, head_dim=dr,
                                                               v_head_dim=dvr), tokens * (2 * qk * 4 + vv * 6) + entries * Hr * dr * dvr * 8, iters=5)
            rec["retention_chunk"]["us_per_token_of_a_request"] = round(rec["retention_chunk"]["us"] / per, 3)
            rec["retention_chunk"]["of_fp32_fma_peak"] = round(fma / (rec["retention_chunk"]["us"] * 1e-6) / (148 * 128 * 1.9e9), 3)
        gated = torch.empty(tokens, vv, device=dev, dtype=bf)
        add("retention_out", lambda: ops.retention_out(o_r, proj_r, 2 * qk + vv, gated, heads=Hr, v_head_dim=dvr, eps=1e-6), tokens * vv * 8)
        # like: the delta rule's recurrence of the closest model, the same state size
        C = 2 * qk + vv
        qkv = torch.randn(tokens, C, device=dev) * 0.1
        dec, beta = torch.rand(tokens, qk, device=dev) * 0.1 + 0.9, torch.rand(tokens, Hr, device=dev)
        state2 = torch.zeros(entries, Hr * dr * dvr + 3 * C, device=dev)
        add("like: delta_scan", lambda: ops.delta_scan(qkv, dec, beta, state2, step, o_r, heads=Hr, kv_heads=Hr, head_dim=dr,
                                                       v_head_dim=dvr), tokens * (C + qk + vv) * 4 + entries * Hr * dr * dvr * 8, iters=5)
        rec["like: delta_scan"]["us_per_token_of_a_request"] = round(rec["like: delta_scan"]["us"] / per, 3)
        out[f"tokens{tokens}_requests{entries}_held{held}"] = rec
        ops.error_check(dev)
    return out


def run(sizes=(2048, 4096), steps: int = 20, warmup: int = 3, kernels: bool = True, parts: bool = True) -> dict:
    torch.cuda.set_device(0)
    pk = peaks()
    points = [("prefill", 1, 2048), ("prefill", 1, 8192), ("prefill", 4, 2048), ("decode", 8, 2048), ("decode", 64, 2048)]
    rec = {"design": "Zisevik", "closest": "Bavutar (hybrid)", "dtype": "bf16", "data": "synthetic", "peaks": pk, "sizes": {}}
    for width in sizes:
        zis, hyb = zisevik_config(width), hybrid_config(width, repeats=2)
        one = {"layer_visits": 8, "zisevik": _throughput(zis, points, steps, warmup), "closest": _throughput(hyb, points, steps, warmup)}
        if parts:
            one["zisevik_parts_ms"] = _parts(zis, 2048, 8)
        if kernels:
            one["kernels"] = _kernels(width, [(2048, 1, 0), (8192, 4, 0), (64, 64, 2048)], pk)
        rec["sizes"][str(width)] = one
    return rec


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--sizes", default="2048,4096")
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-kernels", action="store_true")
    ap.add_argument("--no-parts", action="store_true")
    a = ap.parse_args(argv)
    print(json.dumps(run(tuple(int(s) for s in a.sizes.split(",")), a.steps, max(a.warmup, 3), not a.no_kernels, not a.no_parts)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
