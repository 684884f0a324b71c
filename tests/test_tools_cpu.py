"""Host-side tools: flags, metrics block, cluster collector (with a fake command runner),
comm-model CLI, collective fit, latency table, trace post-processing."""
import json
import os
import subprocess
import sys
import types
import warnings

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_flags_accept_reference_command_line(tmp_path):
    from zorse_b200.config.flags import parse_args_zorse
    from zorse_b200.parallel.schedules import schedule_name_from_flags

    cfg = {"model_name": "tiny_llama", "global_batch_size": 8, "microbatch_size": 2, "sequence_length": 128,
           "autocast_dtype": "bfloat16", "reduce_dtype": "float32", "pipeline_config": []}
    f = tmp_path / "c.json"
    f.write_text(json.dumps(cfg))
    with warnings.catch_warnings(record=True) as w:
        warnings.simplefilter("always")
        a = parse_args_zorse(["--config_file", str(f), "--zero2_pipeline", "--gloo_p2p", "--optimizer_in_backwards",
                              "--hybrid_shard", "--tt_pp", "2", "--iterations", "3"])
    assert any("ignored" in str(x.message) for x in w)
    import torch

    assert a.seq_length == 128 and a.autocast_dtype == torch.bfloat16 and a.global_batch_size == 8
    assert schedule_name_from_flags(a) == "zero2"
    a.flashflex_pipeline = True
    assert schedule_name_from_flags(a) == "flashflex"          # precedence flashflex > zero2
    b = types.SimpleNamespace(two_stage_sync=True, sync_comm=True)
    with pytest.raises(ValueError):
        schedule_name_from_flags(b)
    assert schedule_name_from_flags(types.SimpleNamespace(sync_comm=True)) == "no_overlap"
    assert schedule_name_from_flags(types.SimpleNamespace()) == "layer_major"


def test_metrics_block_and_mfu():
    from zorse_b200.utils import metrics as m

    assert m.clean_gpu_name("NVIDIA B200") == "b200"
    assert m.clean_gpu_name("NVIDIA A100-SXM4-80GB") == "a100x80"
    assert m.clean_gpu_name("NVIDIA H100 NVL") == "h100-nvl"
    fl = m.compute_model_flops(6_738_415_616, 32, 4096, 4096, 64)
    assert fl == pytest.approx(4.5 * (2 * 6_738_415_616 * 4096 + 4 * 32 * 4096 * 4096 ** 2) * 64)
    mfu, tflops = m.compute_mfu(fl, 12000.0, ["b200"], "bfloat16")
    assert 0 < mfu < 1 and tflops == pytest.approx(fl / 12.0 / 1e12)
    per = m.per_gpu_mfu(fl, 12000.0, [3, 1], ["b200", "h100"], "bfloat16")
    assert per[0] > per[1] * 0.5
    s = m.format_summary(global_batch=64, seq=4096, step_ms=12000.0, flops_per_step=fl, gpu_names=["b200"],
                         dtype="bfloat16", max_alloc_gb=[117.0], predicted_ms=12471.0, exposed_comm_ms=0.0, loss=1.5)
    assert m.CSV_HEADER in s and "Throughput: 21845.3 tokens/s" in s and "measured/predicted" in s
    assert s.splitlines()[-1].startswith("64,4096,117.00,117.00,12000.00,21845.33")


def test_cluster_collector_with_fake_runner(tmp_path):
    from zorse_b200.profiler import cluster as C

    hostfile = tmp_path / "hostfile"
    hostfile.write_text("nodeA,~/.ssh/k,/opt/conda.sh,env,~/repo,eth0\nnodeB,,,,~/repo,\n")
    ms = C.read_machine_file(str(hostfile))
    assert [m.hostname for m in ms] == ["nodeA", "nodeB"] and ms[0].socket_ifname == "eth0"
    cmd = C.remote_command(ms[0], "nvidia-smi")
    assert cmd[0] == "ssh" and "-i" in cmd and "conda activate env" in cmd[-1] and "NCCL_SOCKET_IFNAME=eth0" in cmd[-1]

    def runner(cmd, **kw):
        text = " ".join(cmd)
        if "nvidia-smi" in text:
            out = "0, NVIDIA B200, 183359 MiB\n1, NVIDIA B200, 183359 MiB\n" if "nodeA" in text else "0, NVIDIA H100 NVL, 95830 MiB\n"
        elif "--intranode" in text:
            out = "Bandwidth: 742.5 GB/s\nLatency: 0.000054 s\n"
        else:
            out = "Bandwidth: 11.2 GB/s\nLatency: 0.0036 s\n"
        return types.SimpleNamespace(returncode=0, stdout=out, stderr="")

    info = C.collect_cluster_info(ms, runner)
    assert info["total_gpus"] == 3 and [g["global_rank"] for g in info["gpu_list"]] == [0, 1, 2]
    assert info["gpu_list"][2]["name"] == "h100-nvl" and info["global_rank_map"]["2"]["machine"] == "nodeB"
    bw = C.run_bandwidth_test(ms, info, runner)
    assert bw["intranode_bandwidth"]["0"] == 742.5 and bw["intranode_bandwidth"]["1"] == 0.0
    assert bw["internode_bandwidth"]["0"]["1"] == 11.2 and bw["internode_latency"]["0"]["1"] == 0.0036
    info["bandwidth"] = bw
    # the planner reads what the collector writes
    from zorse_b200.planner.cluster import link_bandwidth
    from zorse_b200.planner.partition import build_gpu_graph, partition

    g = info["gpu_list"]
    assert link_bandwidth(info, g[0], g[1]) == 742.5 and link_bandwidth(info, g[2], g[0]) == 11.2
    G = build_gpu_graph(info)
    for alg in ("min_k_cut_split", "min_k_cut_efficient", "clustering"):
        pm = partition(G, 2, alg)
        assert pm["gpu_0"] == pm["gpu_1"] != pm["gpu_2"], alg


def test_collective_fit_and_latency_table(tmp_path):
    from zorse_b200.planner import latency as L
    from zorse_b200.profiler.collectives import fit_switch_model

    R, alpha, bw = 4, 0.05, 600.0
    sizes = [25e6, 100e6, 400e6]
    times = [alpha + (R - 1) / R * s / 1e9 / bw * 1e3 for s in sizes]
    fit = fit_switch_model(sizes, times, R)
    assert fit["alpha_ms"] == pytest.approx(alpha, rel=1e-3) and fit["bandwidth_gbs"] == pytest.approx(bw, rel=1e-3)
    tbl = {}
    L.store(tbl, "llama2_7b", "b200", 4096, "bfloat16", [1.6, 3.4], [4.0, 7.6])
    assert L.lookup(tbl, "llama2_7b", "b200", 4096, "bfloat16", 2).forward == 3.4      # measured value wins
    assert L.lookup(tbl, "llama2_7b", "b200", 4096, "bfloat16", 4).forward == pytest.approx(1.8 * 4 - 0.2)  # linear model
    assert L.lookup(tbl, "llama2_7b", "h100", 4096, "bfloat16", 1) is None
    shipped = L.load_table()
    assert L.lookup(shipped, "llama2_7b", "b200", 4096, "bfloat16", 1) is not None   # profile measured on a B200
    a = L.analytic("llama2_7b", "b200", 4096, 1)
    assert 0.5 < a.forward < 5.0


def test_comm_model_cli_and_param_estimate():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "comm_model.py"), "--cluster_info_file",
                        os.path.join(ROOT, "data", "cluster_info_b200x8.json"), "--ranks", "0,1"],
                       capture_output=True, text=True, cwd=ROOT)
    assert r.returncode == 0 and "all_gather (best model)" in r.stdout
    from zorse_b200.models.param_estimate import estimate

    e = estimate("llama2_7b")
    assert e["parameters_per_layer"] == 202383360 and e["total_parameters"] == 6738415616


def test_trace_postprocessing(tmp_path):
    from zorse_b200.utils.trace import extract_kernel_runtime, stream_busy_and_gaps

    ev = [{"cat": "kernel", "ts": 0, "dur": 100, "args": {"stream": 7}}, {"cat": "kernel", "ts": 150, "dur": 50, "args": {"stream": 7}},
          {"cat": "kernel", "ts": 20, "dur": 30, "args": {"stream": 9}}, {"cat": "cpu_op", "ts": 0, "dur": 999}]
    f = tmp_path / "t.json"
    f.write_text(json.dumps({"traceEvents": ev}))
    assert extract_kernel_runtime(str(f), iterations=2) == pytest.approx(0.09)
    s = stream_busy_and_gaps(str(f))
    assert s[7]["busy_ms"] == pytest.approx(0.15) and s[7]["gap_ms"] == pytest.approx(0.05) and s[9]["kernels"] == 1


def test_trace_streams_are_classified_and_gaps_charged_to_the_other_kind(tmp_path):
    from zorse_b200.utils.trace import classify_streams, stream_overheads

    k = lambda name, ts, dur, s, cat="kernel": {"cat": cat, "name": name, "ts": ts, "dur": dur, "args": {"stream": s}}
    ev = [k("zb::gemm2_bf16_kernel", 0, 100, 7), k("zb::gemm2_bf16_kernel", 300, 100, 7),       # compute gap 100..300
          k("ncclDevKernel_AllGather", 150, 100, 20), k("ncclDevKernel_SendRecv", 180, 40, 21),  # two comm streams overlap
          k("Memcpy HtoD (Pinned -> Device)", 260, 30, 30, "gpu_memcpy"),
          {"cat": "cuda_runtime", "name": "cudaMalloc", "ts": 110, "dur": 20},
          k("zb::rs_adam_kernel<bf16>", 500, 50, 20)]
    kinds = classify_streams(ev)
    assert kinds == {7: "compute", 20: "communication", 21: "communication", 30: "copy"}
    f = tmp_path / "t.json"
    f.write_text(json.dumps({"traceEvents": ev}))
    o = stream_overheads(str(f))
    assert o["compute_gap_ms"] == pytest.approx(0.2)
    assert o["communication_overhead_for_compute"] == pytest.approx(0.1)     # union of the two streams, not 0.14
    assert o["copy_overhead_for_compute"] == pytest.approx(0.03)
    assert o["alloc_overhead_for_compute"] == pytest.approx(0.02)
    assert o["compute_overhead_for_communication"] == pytest.approx(0.1)     # gap 250..500 holds the second GEMM
    assert o["compute_ms"] == pytest.approx(0.4)                             # the 200 us gap counts as busy (< 500 us)


def test_attn_trace_decode_and_phase_stats():
    from zorse_b200.profiler.attn_trace import decode, format_summary, phase_stats, summarize

    words = [(100 << 8) | 1, (150 << 8) | 2, (400 << 8) | 3, (900 << 8) | 4, (1300 << 8) | 5, (2000 << 8) | 1,
             (2040 << 8) | 2, 0, 0]
    ev = decode(words)
    assert ev[0] == (100, "s_ready") and ev[-1] == (2040, "s_loaded") and len(ev) == 7
    st = phase_stats(ev)
    assert st["s_ready->s_loaded"] == {"n": 2, "mean": 45.0, "max": 50, "min": 40, "total": 90}
    assert st["p_half1->s_ready"]["total"] == 700
    summ = summarize([[words, [0, 0, 0]]], 0)
    assert list(summ) == [0] and summ[0]["span"] == 1940
    assert "p_half1->s_ready" in format_summary(summ)


def test_exp2_polynomial_matches_exp2_in_fp32_emulation():
    """The fma-pipe exponential of the attention candidate (csrc/common/ptx.cuh exp2_poly3),
    re-stated in numpy float32: relative error far below a bf16 ulp, exact zero below 2^-126."""
    import numpy as np

    c = np.array([0.9999280571937561, 0.6932610273361206, 0.2426111102104187, 0.05517158284783363], np.float32)
    magic = np.float32(12582912.0)

    def emu(x):
        x = x.astype(np.float32)
        xc = np.maximum(x, np.float32(-126.0))
        t = (xc + magic).astype(np.float32)
        f = (xc - (t - magic)).astype(np.float32)
        p = (c[3] * f + c[2]).astype(np.float32)
        p = (p * f + c[1]).astype(np.float32)
        p = (p * f + c[0]).astype(np.float32)
        r = (p.view(np.int32) + (t.view(np.int32) << np.int32(23))).view(np.float32)
        return np.where(x < -126.0, np.float32(0), r)

    x = np.random.default_rng(0).uniform(-60, 9, 200_000).astype(np.float32)
    rel = np.abs(emu(x) - np.exp2(x.astype(np.float64))) / np.exp2(x.astype(np.float64))
    assert rel.max() < 1e-4
    assert emu(np.array([-np.inf, -1e9, -127.0]))[0] == 0 and emu(np.array([-127.0]))[0] == 0
    assert abs(emu(np.array([0.0]))[0] - 1.0) < 1e-4 and abs(emu(np.array([8.0]))[0] - 256.0) < 0.03

def test_mesh_cli_writes_a_valid_config(capsys):
    import json

    from zorse_b200.config.training_config import parse_pipeline_dict
    from zorse_b200.parallel import mesh

    assert mesh.main(["--pp", "2", "--dp_shard", "2", "--tp", "2", "--model_name", "tiny_llama",
                      "--global_batch_size", "8", "--microbatch_size", "2", "--sequence_length", "32",
                      "--schedule", "1f1b"]) == 0
    cfg = parse_pipeline_dict(json.loads(capsys.readouterr().out))
    assert cfg.world_size == 8 and cfg.tensor_parallel_size == 2 and cfg.schedule == "1f1b"
    assert [s.layer_partition for s in cfg.stages] == [(0, 2), (2, 4)]


def test_candidate_report_parent_side(monkeypatch, capsys):
    """Case list, child-failure handling and the table of the candidate report (no GPU: children are faked)."""
    from zorse_b200.profiler import candidates as C

    assert len(C.CASES) == len(set(C.CASES)) == 30
    fake = {"flash_bwd2:7b": {"case": "flash_bwd2:7b", "agrees": True, "max_diff": 0.01, "tolerance": 0.06, "status_word": 0,
                              "ms_default": 0.9, "ms_candidate": 0.45},
            "norm_bwd2_rms:7b": {"case": "norm_bwd2_rms:7b", "agrees": False, "max_diff": 0.5, "tolerance": 0.03,
                                 "status_word": 3}}
    monkeypatch.setattr(C, "run_child", lambda case, timeout: fake.get(case, {"case": case, "error": "exit code 1: boom"}))
    rc = C.main(["--only", "flash_bwd2:7b,norm_bwd2_rms:7b,norm_fwd2_ln:gqa64"])
    out = capsys.readouterr().out
    assert rc == 1
    assert "| flash_bwd2:7b | yes | 0.01 (0.06) | 0 | 0.900 | 0.450 | 2.00x |" in out
    assert "| norm_bwd2_rms:7b | NO |" in out and "exit code 1: boom" in out
    # a child that prints nothing useful is reported, not raised
    import subprocess as sp
    monkeypatch.undo()
    monkeypatch.setattr(sp, "run", lambda *a, **k: sp.CompletedProcess(a, 3, stdout="", stderr="Traceback\nRuntimeError: x"))
    assert C.run_child("flash_bwd2:7b", 1.0)["error"].startswith("exit code 3: RuntimeError")

def test_package_exports_load_lazily():
    import importlib
    import sys

    import zorse_b200

    assert zorse_b200.__version__
    assert zorse_b200.ParallelDims(tp=2, pp=2).world_size == 4
    assert zorse_b200.parse_pipeline_dict is importlib.import_module("zorse_b200.config.training_config").parse_pipeline_dict
    assert "zorse_b200.trainer" in sys.modules or zorse_b200.Trainer.__name__ == "Trainer"
    import pytest
    with pytest.raises(AttributeError):
        zorse_b200.no_such_name


def test_layer_profile_stores_activation_bytes_and_chain_overhead(tmp_path):
    from zorse_b200.planner import latency as L
    from zorse_b200.planner.memory import estimate_memory_usage, group_memory_bytes
    import torch

    from zorse_b200.profiler.layer import profile_chain

    t: dict = {}
    L.store_activation_bytes(t, "m", "b200", 128, "bfloat16", [100, 180, 260, 350])
    assert L.activation_bytes(t, "m", "b200", 128, "bfloat16", 2) == 180
    assert L.activation_bytes(t, "m", "b200", 128, "bfloat16", 6) == 350 + 2 * 80      # median increase per sequence
    assert L.activation_bytes(t, "m", "a100", 128, "bfloat16", 1) is None
    closed = group_memory_bytes([4], 2, 1000, 1, 128, 64)
    measured = group_memory_bytes([4], 2, 1000, 1, 128, 64, block_activation_bytes=10 * 128 * 64 * 2)
    assert measured - closed == (10 - 2) * 128 * 64 * 2
    e = estimate_memory_usage(10**9, 8, 64, 128, 2, num_shards=4, block_activation_bytes=2**30)
    assert e["training_state_gib"] == pytest.approx(16e9 / 4 / 2**30) and e["activation_gib"] == pytest.approx(1.0)
    assert estimate_memory_usage(10**9, 8, 64, 128, 2, block_activation_bytes=2**30, recompute=False)["activation_gib"] == 8.0
    ch = profile_chain("tiny_llama", 64, torch.float32, blocks=2, iters=2, warmup=1, device=torch.device("cpu"))
    assert ch["blocks"] == 2 and ch["chain_ms"] > 0 and 0.2 < ch["overhead"] < 5.0


def test_status_word_of_the_checking_build_is_decoded(monkeypatch):
    """A bounds report {code 8, site, block} from the checking build reads as a KernelError naming the site."""
    import torch

    from zorse_b200.ops import sm100 as k

    word = torch.tensor([8 | (2 << 4) | (37 << 8)], dtype=torch.int32)
    monkeypatch.setattr(k, "status_word", lambda device=None: word)
    with pytest.raises(k.KernelError, match=r"site 2 \(GEMM epilogue row / column\) in block 37"):
        k.check_status()
    assert int(word.item()) == 0
    word[0] = 5 | (3 << 8)
    with pytest.raises(k.KernelError, match=r"status 5 \(flag wait ran out\) in block 3"):
        k.check_status()


def test_profile_helpers_memcpy_function_time_and_line_fit(tmp_path):
    """Readers of a profiler trace by category and by name, the least-squares line the layer profile stores, and the
    memory line (all zero on a CPU device)."""
    import json

    from zorse_b200.planner import latency
    from zorse_b200.utils import metrics, trace

    ev = [{"cat": "kernel", "name": "zb::gemm2_bf16_kernel<1, 0>", "dur": 1500, "ts": 0},
          {"cat": "kernel", "name": "zb::adam_kernel", "dur": 500, "ts": 2000},
          {"cat": "gpu_memcpy", "name": "Memcpy HtoD (Pinned -> Device)", "dur": 800, "ts": 100},
          {"cat": "cpu_op", "name": "zero.adam", "dur": 4000, "ts": 0},
          {"cat": "cpu_op", "name": "zero.adam", "dur": 2000, "ts": 5000}]
    f = tmp_path / "t.json"
    f.write_text(json.dumps({"traceEvents": ev}))
    assert trace.extract_kernel_runtime(str(f), 2) == pytest.approx(1.0)
    assert trace.extract_memcpy_runtime(str(f), 2) == pytest.approx(0.4)
    assert trace.extract_function_runtime("zero.adam", str(f), 2) == pytest.approx(3.0)
    assert trace.extract_function_runtime("gemm2_bf16_kernel", str(f)) == 0.0
    assert trace.extract_function_runtime("gemm2_bf16_kernel", str(f), exact=False) == pytest.approx(1.5)
    names = ["NVIDIA B200", "NVIDIA B200", "NVIDIA H100", "NVIDIA B200", "NVIDIA H100"]
    assert [trace.first_of_its_model(i, names) for i in range(5)] == [True, False, True, False, False]
    s, c = trace.fit_line([3.0, 5.0, 7.0, 9.0])
    assert s == pytest.approx(2.0) and c == pytest.approx(1.0)
    assert trace.fit_line([4.0]) == (4.0, 0.0)
    with pytest.raises(ValueError):
        trace.fit_line([])
    table = {}
    latency.store(table, "m", "b200", 128, "bfloat16", [3.0, 5.0, 7.0], [6.0, 10.0, 14.0])
    row = table["m"]["b200"]["128"]["bfloat16"]
    assert row[0] == pytest.approx([2.0, 1.0]) and row[1] == pytest.approx([4.0, 2.0])
    lines = []
    st = metrics.print_memory_stats("tag", "cpu", out=lines.append)
    assert st["max_allocated"] == 0.0 and st["tag"] == "tag" and not lines


def test_random_datasets_and_even_split():
    import torch

    from zorse_b200.utils import data

    ds = data.RandomTokenDataset(100, 16, size=10, targets="next", seed=1)
    x, y = ds[3]
    assert len(ds) == 10 and x.dtype == torch.long and torch.equal(y[:-1], x[1:]) and 0 <= int(y[-1]) < 100
    assert torch.equal(data.RandomTokenDataset(100, 16, size=10, seed=1).inputs, ds.inputs)      # same seed, same data
    reg = data.RandomTokenDataset(100, 16, size=4, targets="regression")
    assert reg[0][1].dtype == torch.float32 and float(reg.labels.max()) < 1.0
    with pytest.raises(ValueError):
        data.RandomTokenDataset(100, 16, targets="other")
    img = data.RandomImageDataset(8, size=6, classes=0)
    assert img[0][0].shape == (3, 8, 8) and img[0][1].dtype == torch.float32
    assert data.RandomImageDataset(8, size=6, classes=5).labels.dtype == torch.long
    batches = list(data.get_dataset("tiny_llama", batch_size=4, batches=3, seq_length=8, vocab_size=50))
    assert len(batches) == 3 and batches[0][0].shape == (4, 8) and int(batches[0][0].max()) < 50
    xs, ys = data.split_into(torch.arange(10), torch.arange(10), 4)
    assert [len(a) for a in xs] == [3, 3, 2, 2] and torch.equal(torch.cat(ys), torch.arange(10))
    with pytest.raises(ValueError):
        data.split_into(torch.arange(2), torch.arange(2), 4)


def _groups(pmap):
    out = {}
    for n, p in pmap.items():
        out.setdefault(p, []).append(n)
    return list(out.values())


def test_mixed_graph_weighting_keeps_alike_gpus_together():
    """One switch domain with two GPU generations: bandwidth alone ties every cut (contiguous blocks in rank order,
    which mix the generations here); with the mixed weighting the clustering partitioner puts the four fast and the four
    slow GPUs into one group each."""
    from zorse_b200.planner.partition import build_gpu_graph, partition

    names = ["b200", "h100", "b200", "h100", "b200", "h100", "b200", "h100"]
    data = {"machines": [{"machine": "n0", "machine_index": 0}],
            "gpu_list": [{"id": f"gpu_{i}", "name": n, "memory_total_mib": 183359 if n == "b200" else 81559,
                          "machine": "n0", "global_rank": i} for i, n in enumerate(names)],
            "bandwidth": {"intranode_bandwidth": {"0": 700.0}, "internode_bandwidth": {}}}
    plain = partition(build_gpu_graph(data), 2)
    assert {plain[f"gpu_{i}"] for i in range(4)} == {plain["gpu_0"]}               # ranks 0..3 together: mixed models
    G = build_gpu_graph(data, weighting="mixed", gpu_latency_ms={"b200": 5.3, "h100": 11.0})
    assert G["gpu_0"]["gpu_2"]["weight"] == 100 and G["gpu_0"]["gpu_1"]["weight"] < 90
    mixed = partition(G, 2, "clustering")
    assert len({mixed[f"gpu_{i}"] for i in (0, 2, 4, 6)}) == 1 and len({mixed[f"gpu_{i}"] for i in (1, 3, 5, 7)}) == 1
    assert mixed["gpu_0"] != mixed["gpu_1"]
    # (a minimum cut of a dense graph peels off single GPUs whatever the weights: the cut partitioners are made for
    # clusters whose machines are islands of bandwidth)
    assert sorted(map(len, _groups(partition(G, 2, "min_k_cut_split")))) == [1, 7]
    with pytest.raises(ValueError):
        build_gpu_graph(data, weighting="other")
