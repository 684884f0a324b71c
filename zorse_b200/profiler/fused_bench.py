"""Roofline fractions of the two communication-fused kernels, against NCCL + separate kernels.

    torchrun --nproc-per-node R -m zorse_b200.profiler.fused_bench [--out FILE.json]

For a Llama-2-7B block (202 383 360 bf16 parameters) on R ranks:
* `rs_adam`: time of the fused kernel vs `reduce_scatter_tensor` + the standalone Adam kernel.
  Roofline = slower of NVLink inbound bytes (R-1)/R * N * sizeof(grad) per rank at link
  bandwidth and 0 FLOP compute; the HBM term N/R * 26..28 B is reported next to it.
* `ag_gemm`: fused all-gather + QKV GEMM (4096 tokens) vs `all_gather_into_tensor` + the plain
  GEMM. Roofline = slower of GEMM FLOPs at the measured bf16 peak and inbound bytes
  (R-1)/R * N * 2 at link bandwidth.
Link bandwidth: every fraction is given twice, against the nominal 900 GB/s per direction per GPU and
against 770 GB/s (the peer-copy rate measured on B200 / NVSwitch systems).  `--rs_adam_variants 0,1,2`
times several variants of the reduce-scatter kernel in one run (0 = loads per peer in turn, 1 = all
loads issued up front, 2 = in-switch reduction through the multicast address); `ag_gemm` is timed on
the 2-CTA and the 1-CTA GEMM core and for two chunk sizes.  Times are CUDA-event medians, max over ranks.
"""
from __future__ import annotations

import argparse
import json
import statistics

import torch
import torch.distributed as dist

LINK_GBS = 900.0            # nominal NVLink 5, per direction per GPU
LINK_GBS_MEASURED = 770.0   # peer copy


def _time(fn, pre=None, iters=8, warmup=3):
    ts = []
    for i in range(warmup + iters):
        if pre:
            pre()
        torch.cuda.synchronize()
        dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b)], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if i >= warmup:
            ts.append(float(t.item()))
    return statistics.median(ts)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=None)
    ap.add_argument("--params", type=int, default=202_383_360)
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--rs_adam_variants", default="0", help="comma-separated: 0, 1 (loads up front), 2 (in-switch reduction)")
    ap.add_argument("--peaks", default=None, help="JSON with measured hbm_gbs / bf16_tflops of this machine")
    a = ap.parse_args(argv)
    import torch.distributed._symmetric_memory as symm

    from zorse_b200.ops import sm100 as k
    from zorse_b200.parallel.groups import dist_init
    from zorse_b200.profiler.kernel_bench import _peaks

    dev = dist_init()
    rank, R = dist.get_rank(), dist.get_world_size()
    peaks = _peaks(a.peaks)
    variants = [int(v) for v in a.rs_adam_variants.split(",")]
    q = 64 * R
    n = (a.params + q - 1) // q * q
    sn = n // R
    res = {"R": R, "params": n, "link_gbs": LINK_GBS, "link_gbs_measured": LINK_GBS_MEASURED, "peaks": peaks}
    hyper = dict(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0)

    # ---------------------------------------------------------------- rs_adam
    for variant in variants:
      k.set_rs_adam_variant(variant)
      for gdt, name in ((torch.bfloat16, "bf16"), (torch.float32, "fp32")):
        grad = symm.empty(n, dtype=gdt, device=dev)
        flags = symm.empty(64, dtype=torch.int32, device=dev)
        grad.normal_()
        flags.zero_()
        torch.cuda.synchronize()
        hg, hf = symm.rendezvous(grad, dist.group.WORLD), symm.rendezvous(flags, dist.group.WORLD)
        master, m, v = (torch.zeros(sn, device=dev) for _ in range(3))
        p16 = torch.empty(sn, dtype=torch.bfloat16, device=dev)
        counter = torch.zeros(1, dtype=torch.int32, device=dev)
        g_sh = torch.empty(sn, dtype=gdt, device=dev)
        epoch = [0]

        mc = int(getattr(hg, "multicast_ptr", 0) or 0)
        if variant == 2 and mc == 0:
            res[f"rs_adam_v2_{name}"] = {"skipped": "no NVLS multicast address for this group"}
            continue

        def fused():
            epoch[0] += 1
            kw = dict(step=epoch[0], grad_scale=1.0, grad_f32=gdt == torch.float32, epoch=epoch[0], counter=counter,
                      **hyper)
            if variant == 2:
                k.rs_adam_nvls(mc, [int(x) for x in hf.buffer_ptrs], R, rank, sn, master, m, v, p16, **kw)
            else:
                k.rs_adam([int(x) for x in hg.buffer_ptrs], [int(x) for x in hf.buffer_ptrs], R, rank, sn, master, m,
                          v, p16, **kw)
            k.wait_flags(flags, R, 1, epoch[0])

        def library():
            dist.reduce_scatter_tensor(g_sh, grad)
            k.adam_step(master, m, v, g_sh, p16, step=1, grad_scale=1.0, **hyper)

        t_f, t_l = _time(fused), _time(library)
        k.check_status()
        gb = grad.element_size()
        inbound = (R - 1) / R * n * gb
        if variant == 2:
            inbound = n / R * gb * 1.0      # the switch delivers the sum: one slice's worth of bytes comes in
        link_ms = inbound / (LINK_GBS * 1e9) * 1e3
        link_ms_meas = inbound / (LINK_GBS_MEASURED * 1e9) * 1e3
        # optimizer state read + written (fp32 master, two moments: 24 B; bf16 copy written: 2 B) and the
        # gradient slices this rank reads (its own from HBM)
        hbm_ms = (sn * 26 + sn * gb) / (peaks["hbm_gbs"] * 1e9) * 1e3
        res[f"rs_adam_v{variant}_{name}"] = {
            "fused_ms": t_f, "nccl_plus_adam_ms": t_l, "nvlink_ms_at_900": link_ms, "nvlink_ms_at_770": link_ms_meas,
            "hbm_term_ms": hbm_ms, "frac_of_roofline_900": max(link_ms, hbm_ms) / t_f,
            "frac_of_roofline_770": max(link_ms_meas, hbm_ms) / t_f}
        dist.barrier()
    k.set_rs_adam_variant(0)

    # ---------------------------------------------------------------- ag_gemm (QKV of a 7B block)
    N, K, M = 12288, 4096, a.tokens
    full = symm.empty(n, dtype=torch.bfloat16, device=dev)
    vflags = symm.empty(64, dtype=torch.int32, device=dev)
    full.normal_(std=0.02)
    vflags.zero_()
    torch.cuda.synchronize()
    hfull = symm.rendezvous(full, dist.group.WORLD)
    symm.rendezvous(vflags, dist.group.WORLD)
    x = torch.randn(M, K, device=dev).to(torch.bfloat16)
    out = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
    shard = full[rank * sn:(rank + 1) * sn].clone()
    gathered = torch.empty(n, dtype=torch.bfloat16, device=dev)
    off = 4096  # the norm weight precedes the QKV weight in a block's flat layout
    shard_ptrs = [int(hfull.buffer_ptrs[qq]) + qq * sn * 2 for qq in range(R)]

    def library_ag():
        dist.all_gather_into_tensor(gathered, shard)
        k.gemm(x, gathered[off:off + N * K].view(N, K), out)

    def gemm_only():
        k.gemm(x, full[off:off + N * K].view(N, K), out)

    t_l, t_g = _time(library_ag), _time(gemm_only)
    inbound = (R - 1) / R * n * 2
    link_ms, link_ms_meas = inbound / (LINK_GBS * 1e9) * 1e3, inbound / (LINK_GBS_MEASURED * 1e9) * 1e3
    gemm_ms = 2.0 * M * N * K / (peaks["bf16_tflops"] * 1e12) * 1e3
    res["ag_gemm"] = {"nccl_plus_gemm_ms": t_l, "gemm_alone_ms": t_g, "nvlink_ms_at_900": link_ms,
                      "nvlink_ms_at_770": link_ms_meas, "gemm_roofline_ms": gemm_ms}
    import os

    for kern in ("2cta", "1cta"):
        for chunk in (1 << 15, 1 << 18):
            os.environ["ZORSE_AG_GEMM"] = kern
            cps = (sn * 2 + chunk - 1) // chunk
            cflags = torch.zeros(R * cps, dtype=torch.int32, device=dev)
            ep = [0]

            def fused_ag():
                ep[0] += 1
                k.ag_gemm(x, full, off, (N, K), out, shard_ptrs=shard_ptrs, R=R, r=rank, shard_elems=sn,
                          chunk_bytes=chunk, chunk_flags=cflags, epoch=ep[0], version_flags=vflags[2 * R:], need_version=0)

            t_f = _time(fused_ag)
            k.check_status()
            res["ag_gemm"][f"{kern}_chunk{chunk >> 10}k"] = {
                "fused_ms": t_f, "frac_of_roofline_900": max(link_ms, gemm_ms) / t_f,
                "frac_of_roofline_770": max(link_ms_meas, gemm_ms) / t_f}
    os.environ.pop("ZORSE_AG_GEMM", None)
    if rank == 0:
        print(json.dumps(res, indent=1))
        if a.out:
            with open(a.out, "w") as f:
                json.dump(res, f, indent=1)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
