"""Throughput / MFU / memory summary printed at the end of a run.

Definitions follow the reference (utils/train_utils.py:371-446, 556-734):
    tokens/s   = global_batch_size * seq_length / (avg_iteration_ms / 1000)
    FLOPs/step = 4.5 * (2 * P * S + 4 * L * H * S^2) * global_batch     (1 fwd + 2 bwd + 1 recompute + 0.5)
    MFU        = FLOPs/step / step_time / sum over GPUs of peak[dtype][gpu]
and the CSV line keeps the reference's header.  The peak table gains bfloat16 rows and the
B200 (nominal dense 2250 TFLOP/s bf16/fp16); iteration time is the max over ranks.
"""
from __future__ import annotations

from typing import Optional

import torch

GPU_TFLOPS = {
    "float16": {"b200": 2250.0, "h100-nvl": 835.0, "h100": 989.0, "l40s": 362.0, "a100x80": 312.0, "a100": 312.0,
                "a6000": 155.0, "l4": 120.0, "a10g": 125.0, "v100": 125.0, "t4": 65.0, "p40": 12.0},
    "float32": {"b200": 80.0, "h100-nvl": 60.0, "h100": 67.0, "l40s": 91.6, "a100x80": 19.5, "a100": 19.5,
                "a6000": 38.7, "l4": 30.3, "a10g": 31.2, "v100": 15.7, "t4": 8.1, "p40": 12.0},
}
GPU_TFLOPS["bfloat16"] = dict(GPU_TFLOPS["float16"])

CSV_HEADER = ("Batch Size,Seq_Len,Min_Allocated,Max_Allocated,Latency,Throughput,Avg_Compute_Utilization,"
              "Mem_Utilization,Alloc_Overhead,MFU,TFLOPs")


def clean_gpu_name(name: str) -> str:
    """'NVIDIA B200' -> 'b200' (last word, lower case, with aliases; reference utils/comm.py:70-88)."""
    n = name.strip().lower()
    if "a100" in n:
        return "a100x80" if "80" in n else "a100"
    if "h100" in n:
        return "h100-nvl" if "nvl" in n else "h100"
    return n.replace("nvidia", "").strip().split(" ")[-1].split("-")[0] if n else "cpu"


def compute_model_flops(total_params: int, num_layers: int, hidden: int, seq: int, global_batch: int,
                        recompute: bool = True) -> float:
    factor = 4.5 if recompute else 3.5
    return factor * (2.0 * total_params * seq + 4.0 * num_layers * hidden * seq * seq) * global_batch


def compute_mfu(flops_per_step: float, step_ms: float, gpu_names: list[str], dtype: str) -> tuple[float, float]:
    """(MFU, achieved TFLOP/s over the whole job)."""
    table = GPU_TFLOPS.get(dtype, GPU_TFLOPS["bfloat16"])
    peak = sum(table.get(g, table["b200"]) for g in gpu_names) or 1.0
    achieved = flops_per_step / (step_ms / 1e3) / 1e12
    return achieved / peak, achieved


def per_gpu_mfu(flops_per_step: float, step_ms: float, shares: list[float], gpu_names: list[str], dtype: str):
    """MFU of each GPU of a heterogeneous job: its FLOPs share (proportional to the layers x
    microbatches it runs) against its own peak (reference utils/train_utils.py:449-506)."""
    table = GPU_TFLOPS.get(dtype, GPU_TFLOPS["bfloat16"])
    tot = sum(shares) or 1.0
    return [flops_per_step * s / tot / (step_ms / 1e3) / 1e12 / table.get(g, table["b200"])
            for s, g in zip(shares, gpu_names)]


def memory_stats(device) -> dict:
    if torch.device(device).type != "cuda":
        return {"allocated_gb": 0.0, "max_allocated_gb": 0.0, "max_reserved_gb": 0.0, "alloc_retries": 0}
    st = torch.cuda.memory_stats(device)
    return {"allocated_gb": torch.cuda.memory_allocated(device) / 2**30,
            "max_allocated_gb": torch.cuda.max_memory_allocated(device) / 2**30,
            "max_reserved_gb": torch.cuda.max_memory_reserved(device) / 2**30,
            "alloc_retries": st.get("num_alloc_retries", 0)}


def print_memory_stats(tag: str, device, rank: int = 0, skip: bool = False, out=print) -> dict:
    """One line per call with allocated / peak allocated / peak reserved memory in GiB and as a share of the device,
    and the allocator's retry count (a non-zero count means the step ran against the memory limit); returns the
    figures (reference utils/profile.py:16-48).  On a CPU device, or with `skip`, everything is zero and nothing
    is printed."""
    st = {"tag": tag, "allocated": 0.0, "max_allocated": 0.0, "max_reserved": 0.0, "cuda_malloc_retries": 0}
    if skip or torch.device(device).type != "cuda":
        return st
    torch.cuda.synchronize(device)
    m = memory_stats(device)
    total = torch.cuda.get_device_properties(device).total_memory / 2**30
    st.update(allocated=m["allocated_gb"], max_allocated=m["max_allocated_gb"], max_reserved=m["max_reserved_gb"],
              cuda_malloc_retries=m["alloc_retries"])
    out(f"rank {rank} {tag}: {st['allocated']:.2f} GiB allocated ({100 * st['allocated'] / total:.2f}%), "
        f"{st['max_allocated']:.2f} GiB max allocated ({100 * st['max_allocated'] / total:.2f}%), "
        f"{st['max_reserved']:.2f} GiB max reserved ({100 * st['max_reserved'] / total:.2f}%), "
        f"{st['cuda_malloc_retries']} cuda malloc retries")
    return st


def format_summary(*, global_batch: int, seq: int, step_ms: float, flops_per_step: float, gpu_names: list[str],
                   dtype: str, max_alloc_gb: list[float], predicted_ms: Optional[float] = None,
                   exposed_comm_ms: Optional[float] = None, loss: Optional[float] = None, flashflex_ga: int = 1) -> str:
    gb = global_batch * max(flashflex_ga, 1)
    tput = gb * seq / (step_ms / 1e3)
    mfu, tflops = compute_mfu(flops_per_step, step_ms, gpu_names, dtype)
    lines = [
        "===== zorse-b200 run summary =====",
        f"GPUs: {len(gpu_names)} ({', '.join(sorted(set(gpu_names)))})",
        f"Max allocated memory per GPU (GB): min {min(max_alloc_gb):.2f} max {max(max_alloc_gb):.2f} "
        f"total {sum(max_alloc_gb):.2f}",
        f"Time per step (max over ranks): {step_ms:.2f} ms",
        f"Throughput: {tput:.1f} tokens/s",
        f"MFU: {100 * mfu:.2f}%   achieved {tflops:.1f} TFLOP/s",
    ]
    if predicted_ms is not None:
        lines.append(f"Planner-predicted step time: {predicted_ms:.2f} ms (measured/predicted = {step_ms / predicted_ms:.3f})")
    if exposed_comm_ms is not None:
        lines.append(f"Exposed communication: {exposed_comm_ms:.2f} ms/step")
    if loss is not None:
        lines.append(f"Loss (last step): {loss:.4f}")
    lines.append(CSV_HEADER)
    lines.append(f"{gb},{seq},{min(max_alloc_gb):.2f},{max(max_alloc_gb):.2f},{step_ms:.2f},{tput:.2f},"
                 f"{100 * mfu:.2f},0.00,0.00,{100 * mfu:.2f},{tflops:.2f}")
    return "\n".join(lines)
