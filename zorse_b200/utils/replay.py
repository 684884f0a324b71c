"""Deterministic-replay check (debug): run one training step twice from the same state and
compare every unit's master weights and Adam moments bit by bit.

A difference means that something in the step depends on timing: an unordered cross-stream
access, a reduction whose order varies, a buffer read before it was filled.  The kernels of this
repository reduce in a fixed order (fixed peer order in the fused reduce-scatter, two-step
column sums) with one known exception, the attention backward's fp32 `red.global.add`
accumulation of dQ, whose order depends on CTA scheduling; with it the check reports the units
that differ and by how much instead of failing outright (`tolerance`).
The reference has no counterpart (it has no race detection of any kind).
"""
from __future__ import annotations

import torch


def snapshot(trainer) -> list[dict]:
    trainer.synchronize()
    out = []
    for st in trainer.stages:
        for u in st.engine.units:
            t = u.state_tensors()
            out.append({"unit": u, "master": t["master"].detach().clone(), "m": t["m"].detach().clone(),
                        "v": t["v"].detach().clone(), "step": u.step_count})
    return out


def restore(trainer, snap: list[dict]) -> None:
    for e in snap:
        e["unit"].load_state(e["master"], e["m"], e["v"], e["step"])
    trainer.synchronize()


def compare(a: list[dict], b: list[dict]) -> list[dict]:
    """Units whose state differs between two snapshots, with the largest absolute difference."""
    diffs = []
    for x, y in zip(a, b):
        worst = 0.0
        for k in ("master", "m", "v"):
            if not torch.equal(x[k], y[k]):
                worst = max(worst, float((x[k].float() - y[k].float()).abs().max()))
        if worst > 0.0 or x["step"] != y["step"]:
            diffs.append({"gid": x["unit"].gid, "kind": x["unit"].layer.kind, "max_abs_diff": worst})
    return diffs


def replay_check(trainer, inputs, targets, tolerance: float = 0.0) -> dict:
    """Steps once, rewinds, steps again. Leaves the trainer one step further (second run's state).
    Returns {"identical", "within_tolerance", "differing_units", "loss"}."""
    before = snapshot(trainer)
    step0 = trainer.step_idx
    l1 = trainer.train_step(inputs, targets)
    first = snapshot(trainer)
    l1 = None if l1 is None else float(l1)
    restore(trainer, before)
    trainer.step_idx = step0
    l2 = trainer.train_step(inputs, targets)
    second = snapshot(trainer)
    l2 = None if l2 is None else float(l2)
    diffs = compare(first, second)
    return {"identical": not diffs and l1 == l2,
            "within_tolerance": all(d["max_abs_diff"] <= tolerance for d in diffs),
            "differing_units": diffs, "loss": (l1, l2)}
