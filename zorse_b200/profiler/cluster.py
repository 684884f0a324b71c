"""Cluster collector: machines, GPUs, bandwidths -> cluster_info.json.

Hostfile: one CSV line per machine, `hostname,ssh_key_path,conda_sh,conda_env,repo_path,NCCL_SOCKET_IFNAME`
(reference README.md:27-30, utils/collect_cluster_utils.py:7-66).  A hostname of `localhost`
(or a missing hostfile) runs everything on this machine without ssh.  GPUs are listed with
`nvidia-smi --query-gpu=index,name,memory.total`; global ranks follow hostfile order.  The
intra-node probe runs `benchmark_gpu_bandwidth.py --intranode` under torchrun on each machine;
the inter-node probe runs it `--internode` on machine pairs (all pairs, or one representative
pair per (region, GPU-set) class with `optimize_internode`).  On a machine with NVSwitch the
collector also fits all-gather / reduce-scatter alpha and bandwidth per group size
(`collective_fit`) with `run_comm_profiling`.
"""
from __future__ import annotations

import json
import os
import re
import shlex
import subprocess
import sys
from dataclasses import dataclass
from typing import Optional

from ..utils.metrics import clean_gpu_name


@dataclass
class Machine:
    hostname: str
    ssh_key: str = ""
    conda_sh: str = ""
    conda_env: str = ""
    repo_path: str = ""
    socket_ifname: str = ""

    @property
    def local(self) -> bool:
        return self.hostname in ("localhost", "127.0.0.1", "")


def read_machine_file(path: Optional[str]) -> list[Machine]:
    if not path or not os.path.exists(path):
        return [Machine("localhost", repo_path=os.getcwd())]
    out = []
    with open(path) as f:
        for line in f:
            line = line.strip()
            if not line or line.startswith("#"):
                continue
            parts = [p.strip() for p in line.split(",")]
            parts += [""] * (6 - len(parts))
            out.append(Machine(*parts[:6]))
    return out


def remote_command(m: Machine, inner: str, env: Optional[dict] = None) -> list[str]:
    """argv that runs `inner` in the machine's repo and environment (ssh unless local)."""
    pre = []
    if m.repo_path:
        pre.append(f"cd {shlex.quote(os.path.expanduser(m.repo_path)) if m.local else m.repo_path}")
    if m.conda_sh:
        pre.append(f"source {m.conda_sh}")
    if m.conda_env:
        pre.append(f"conda activate {m.conda_env}")
    envs = dict(env or {})
    if m.socket_ifname:
        envs.setdefault("NCCL_SOCKET_IFNAME", m.socket_ifname)
        envs.setdefault("GLOO_SOCKET_IFNAME", m.socket_ifname)
    envstr = " ".join(f"{k}={shlex.quote(str(v))}" for k, v in envs.items())
    cmd = " && ".join(pre + [f"{envstr} {inner}".strip()])
    if m.local:
        return ["bash", "-lc", cmd]
    ssh = ["ssh", "-o", "StrictHostKeyChecking=no"]
    if m.ssh_key:
        ssh += ["-i", os.path.expanduser(m.ssh_key)]
    return ssh + [m.hostname, cmd]


def parse_nvidia_smi(text: str) -> list[dict]:
    gpus = []
    for line in text.strip().splitlines():
        parts = [p.strip() for p in line.split(",")]
        if len(parts) < 3 or not parts[0].isdigit():
            continue
        mem = re.sub(r"[^0-9]", "", parts[2])
        gpus.append({"index": int(parts[0]), "name": clean_gpu_name(parts[1]), "memory_total_mib": int(mem or 0)})
    return gpus


def get_gpu_info(m: Machine, runner=subprocess.run) -> list[dict]:
    cmd = remote_command(m, "nvidia-smi --query-gpu=index,name,memory.total --format=csv,noheader")
    r = runner(cmd, capture_output=True, text=True, timeout=60)
    if r.returncode != 0:
        return []
    return parse_nvidia_smi(r.stdout)


def collect_cluster_info(machines: list[Machine], runner=subprocess.run) -> dict:
    info = {"machines": [], "total_gpus": 0, "gpu_list": [], "global_rank_map": {}}
    rank = 0
    for mi, m in enumerate(machines):
        gpus = get_gpu_info(m, runner)
        entry = {"machine": m.hostname, "num_gpus": len(gpus), "gpus": [], "machine_index": mi}
        for g in gpus:
            rec = {**g, "id": f"gpu_{rank}", "machine": m.hostname, "global_rank": rank}
            entry["gpus"].append(rec)
            info["gpu_list"].append(rec)
            info["global_rank_map"][str(rank)] = {"machine": m.hostname, "local_rank": g["index"], "machine_index": mi}
            rank += 1
        info["machines"].append(entry)
    info["total_gpus"] = rank
    return info


_BW = re.compile(r"Bandwidth:\s*([0-9.eE+-]+)\s*G[bB]/s")
_LAT = re.compile(r"Latency:\s*([0-9.eE+-]+)\s*(?:s|ms)")


def parse_bandwidth_output(text: str) -> tuple[Optional[float], Optional[float]]:
    b, l = _BW.search(text), _LAT.search(text)
    return (float(b.group(1)) if b else None, float(l.group(1)) if l else None)


def intranode_command(m: Machine, num_gpus: int, port: int = 12355, fast: bool = True, msg: int = 10_000_000) -> list[str]:
    inner = (f"{sys.executable if m.local else 'python'} -m torch.distributed.run --nnodes=1 --nproc-per-node {num_gpus} "
             f"--master-addr 127.0.0.1 --master-port {port} benchmark_gpu_bandwidth.py --intranode "
             f"{'--fast_intra ' if fast else ''}--send_msg_size {msg}")
    return remote_command(m, inner)


def internode_commands(a: Machine, b: Machine, port: int = 12346, msg: int = 10_000_000) -> list[list[str]]:
    cmds = []
    for node_rank, m in enumerate((a, b)):
        inner = (f"{sys.executable if m.local else 'python'} -m torch.distributed.run --nnodes=2 --node-rank {node_rank} "
                 f"--nproc-per-node 1 --master-addr {a.hostname} --master-port {port} benchmark_gpu_bandwidth.py "
                 f"--internode --send_msg_size {msg}")
        cmds.append(remote_command(m, inner, {"NCCL_IB_DISABLE": "1"}))
    return cmds


def machine_class(entry: dict, region: str = "") -> tuple:
    return (region, tuple(sorted(g["name"] for g in entry["gpus"])))


def run_bandwidth_test(machines: list[Machine], info: dict, runner=subprocess.run, optimize_internode: bool = False,
                       fast_intra: bool = True) -> dict:
    bw = {"internode_bandwidth": {}, "intranode_bandwidth": {}, "internode_latency": {}, "intranode_latency": {}}
    for mi, (m, entry) in enumerate(zip(machines, info["machines"])):
        if entry["num_gpus"] < 2:
            bw["intranode_bandwidth"][str(mi)], bw["intranode_latency"][str(mi)] = 0.0, 0.0
            continue
        r = runner(intranode_command(m, entry["num_gpus"], fast=fast_intra), capture_output=True, text=True, timeout=900)
        b, l = parse_bandwidth_output(r.stdout + r.stderr)
        bw["intranode_bandwidth"][str(mi)] = b or 0.0
        bw["intranode_latency"][str(mi)] = l or 0.0
    n = len(machines)
    classes = [machine_class(e) for e in info["machines"]]
    cache: dict = {}
    for i in range(n):
        for j in range(i + 1, n):
            key = (classes[i], classes[j]) if optimize_internode else (i, j)
            if key not in cache:
                procs = [subprocess.Popen(c, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
                         for c in internode_commands(machines[i], machines[j])] if runner is subprocess.run else None
                if procs is None:
                    out = runner(internode_commands(machines[i], machines[j])[0], capture_output=True, text=True).stdout
                else:
                    out = "".join(p.communicate(timeout=900)[0] for p in procs)
                cache[key] = parse_bandwidth_output(out)
            b, l = cache[key]
            bw["internode_bandwidth"].setdefault(str(i), {})[str(j)] = b or 0.0
            bw["internode_latency"].setdefault(str(i), {})[str(j)] = l or 0.0
    return bw


def fit_collectives_locally(num_gpus: int, num_parameters: int, runner=subprocess.run, port: int = 12345) -> dict:
    """alpha / bandwidth of all-gather and reduce-scatter for R = 2, 4, 8 on this machine."""
    fit = {"all_gather": {}, "reduce_scatter": {}}
    for R in (2, 4, 8):
        if R > num_gpus:
            break
        out = f"/tmp/zorse_fit_{R}.json"
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={R}", "--master-addr",
               "127.0.0.1", "--master-port", str(port), "-m", "zorse_b200.profiler.run_comm_profiling",
               "--num_parameters", str(num_parameters), "--fit", "--output", out]
        r = runner(cmd, capture_output=True, text=True, timeout=900)
        if r.returncode == 0 and os.path.exists(out):
            with open(out) as f:
                d = json.load(f).get("fit", {})
            for k in fit:
                fit[k].update(d.get(k, {}))
    return fit
