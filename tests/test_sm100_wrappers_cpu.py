"""Every Python wrapper of the kernel library, called on CPU tensors against a stand-in library that only
records which entry point was reached: catches mistakes in argument marshalling, names and version
selection of code that otherwise only runs on a GPU.  (What the kernels compute is tested on the GPU.)"""
import pytest
import torch

from zorse_b200.ops import sm100 as k


class FakeLib:
    def __init__(self):
        self.calls = []

    def __getattr__(self, name):
        def f(*args):
            self.calls.append((name, len(args)))
            if name.endswith("partial_rows"):
                return 8
            if name.endswith("stats_floats"):
                return 2 * 128 * 4
            if name.endswith("trace_warps"):
                return 10
            if name.endswith("trace_events"):
                return 16
            if name.endswith("probe_count"):
                return 64
            return 0
        return f


def c_prototypes():
    """{entry point: number of parameters} read from the CUDA sources."""
    import pathlib
    import re

    root = pathlib.Path(__file__).resolve().parent.parent / "csrc"
    out = {}
    for f in root.rglob("*.cu"):
        text = f.read_text()
        for m in re.finditer(r"\b(?:int|void)\s+(zb_\w+)\s*\(([^)]*)\)\s*\{", text):
            params = m.group(2).strip()
            out[m.group(1)] = 0 if params in ("", "void") else params.count(",") + 1
    return out


@pytest.fixture
def lib(monkeypatch):
    fake = FakeLib()
    monkeypatch.setattr(k, "_lib", fake)
    monkeypatch.setattr(k, "_bf16", lambda t, name: None)
    monkeypatch.setattr(k, "status_word", lambda device=None: torch.zeros(1, dtype=torch.int32))
    monkeypatch.setattr(k, "_stream", lambda: None)
    monkeypatch.setattr(k, "_attn_scratch", {})
    monkeypatch.setattr(k, "_attn_scratch2", {})
    yield fake
    protos = c_prototypes()
    for name, nargs in fake.calls:
        assert name in protos, f"{name} is not defined in csrc/"
        assert nargs == protos[name], f"{name}: called with {nargs} arguments, the C function takes {protos[name]}"


def bf(*shape):
    return torch.zeros(*shape, dtype=torch.bfloat16)


def names(lib):
    return [c[0] for c in lib.calls]


def test_gemm_dispatch(lib, monkeypatch):
    a, w, out = bf(512, 256), bf(384, 256), bf(512, 384)
    k.gemm(a, w, out)
    k.gemm(a, w, out, accumulate=True, kernel="2cta_accpf")
    k.gemm(a[:100], w, out[:100])                        # below the 2-CTA tile: single-CTA kernel
    k.gemm(a, w, out, kernel="1cta", act="gelu", bias=bf(384), addend=bf(512, 384))
    monkeypatch.setattr(k, "GEMM_ACC_PREFETCH", True)
    k.gemm(a, w, out, accumulate=True)
    k.gemm(a, w, out)
    assert names(lib) == ["zb_gemm2_bf16", "zb_gemm2_accpf_bf16", "zb_gemm_bf16", "zb_gemm_bf16",
                          "zb_gemm2_accpf_bf16", "zb_gemm2_bf16"]
    with pytest.raises(TypeError):
        k.gemm(a, w, torch.zeros(512, 384, dtype=torch.float16))


def test_norm_and_attention_versions(lib):
    x, w, b = bf(64, 256), bf(256), bf(256)
    y, st = k.norm_fwd(x, w, None, 1e-5, False)
    k.norm_fwd(x, w, b, 1e-5, True, version=2)
    dw, db = torch.zeros(256), torch.zeros(256)
    k.norm_bwd(x, x, w, st, None, dw, None, False, version=1)
    k.norm_bwd(x, x, w, st, x, dw, db, True)                 # version 2 is the default
    B, S, Hq, Hkv, D = 1, 128, 4, 2, 64
    qkv, do = bf(B * S, (Hq + 2 * Hkv) * D), bf(B * S, Hq * D)
    out, lse = k.flash_fwd(qkv, B, S, Hq, Hkv, D)
    k.flash_fwd(qkv, B, S, Hq, Hkv, D, version=2)
    k.flash_fwd(qkv, B, S, Hq, Hkv, D, True, 32, version=4, flags=2,
                trace=k.flash_fwd4_trace_buffer("cpu", 2), trace_ctas=2)
    k.flash_bwd(do, qkv, out, lse, B, S, Hq, Hkv, D, version=1)
    k.flash_bwd(do, qkv, out, lse, B, S, Hq, Hkv, D)                     # version 3 is the default
    k.flash_bwd(do, qkv, out, lse, B, S, Hq, Hkv, D, version=2, trace=k.flash_bwd2_trace_buffer("cpu", 1), trace_ctas=1)
    got = [n for n in names(lib) if not n.endswith(("partial_rows", "stats_floats", "trace_warps", "trace_events"))]
    assert got == ["zb_norm_fwd", "zb_norm_fwd2", "zb_norm_bwd", "zb_norm_bwd2", "zb_flash_fwd", "zb_flash_fwd2",
                   "zb_flash_fwd4", "zb_flash_bwd", "zb_flash_bwd3", "zb_flash_bwd2"]
    assert out.shape == (B * S, Hq * D) and lse.shape == (B, Hq, S) and y.shape == x.shape and st.shape == (64, 2)


def test_elementwise_loss_optimizer(lib):
    gu = bf(32, 512)
    k.swiglu_fwd(gu)
    k.swiglu_bwd(gu, bf(32, 256))
    k.act_fwd(gu, k.ACT_GELU_TANH)
    k.act_bwd(gu, gu, k.ACT_RELU)
    k.rope_(bf(32, 6 * 64), torch.zeros(32, 64), 32, 4, 64)
    ids = torch.zeros(32, dtype=torch.long)
    k.embedding_fwd(ids, bf(100, 64), bf(40, 64), 32, 2)
    k.embedding_bwd(ids, bf(32, 64), torch.zeros(100, 64), torch.zeros(40, 64), 32, 2)
    k.cross_entropy(bf(32, 100), ids, 1.0, dlogits=bf(32, 100))
    n = 1024
    k.adam_step(torch.zeros(n), torch.zeros(n), torch.zeros(n), bf(n), bf(n), lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8,
                weight_decay=0.0, step=1)
    k.colsum_accumulate(bf(32, 64), torch.zeros(64))
    assert len(lib.calls) >= 10 and all(isinstance(c[1], int) for c in lib.calls)


def test_fused_collective_wrappers(lib):
    R, rows, H = 2, 256, 256
    ptrs = [1 << 20, 2 << 20]
    counter = torch.zeros(1, dtype=torch.int32)
    flags = torch.zeros(64, dtype=torch.int32)
    hyper = dict(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0, step=1, grad_scale=1.0, grad_f32=False,
                 epoch=1, counter=counter)
    sh = torch.zeros(1024)
    k.rs_adam(ptrs, ptrs, R, 0, 1024, sh, sh, sh, bf(1024), **hyper)
    k.rs_adam_nvls(1 << 30, ptrs, R, 0, 1024, sh, sh, sh, bf(1024), p16_mc=(1 << 31), **hyper)
    k.set_rs_adam_variant(1)
    k.wait_flags(flags, R, 2, 1)
    k.peer_pull(ptrs[1], bf(1024), 2048)
    k.ag_gemm(bf(64, 128), bf(8192 * 4), 64, (256, 128), bf(64, 256), shard_ptrs=ptrs, R=R, r=0, shard_elems=16384,
              chunk_bytes=4096, chunk_flags=torch.zeros(16, dtype=torch.int32), epoch=1, version_flags=flags, need_version=0)
    k.gemm_rs(bf(R * rows, 128), bf(H, 128), b_mn=False, dst_ptrs=ptrs, flag_ptrs=ptrs, flag_index=1, epoch=3,
              counter=counter, ldc=H)
    k.gemm_rs(bf(R * rows, 128), bf(128, H), b_mn=True, dst_ptrs=ptrs, flag_ptrs=ptrs, flag_index=1, epoch=3,
              counter=counter, ldc=H)
    out = k.rs_finish(bf(R * rows * H), flags[:R], R, rows, H, 3, bf(rows, H), resid=bf(rows, H), bias=bf(H))
    assert out.shape == (rows, H)
    st = torch.zeros(rows, 2)
    k.tp_norm_push(x=bf(rows, H), w=bf(H), b=None, eps=1e-5, layernorm=False, y_local=bf(rows, H), dst_ptrs=ptrs,
                   flag_ptrs=ptrs, flag_index=17, epoch=1, stats=st, counter=counter)
    k.tp_norm_push(slots=bf(R * rows * H), in_flags=flags[:R], in_epoch=3, resid=bf(rows, H), bias=bf(H), h_out=bf(rows, H),
                   w=bf(H), b=bf(H), eps=1e-5, layernorm=True, y_local=bf(rows, H), dst_ptrs=ptrs, flag_ptrs=ptrs,
                   flag_index=17, epoch=2, stats=st, counter=counter)
    k.tp_push(bf(rows, H), ptrs, ptrs, 16, 1, counter)
    assert names(lib) == ["zb_rs_adam", "zb_rs_adam_nvls", "zb_set_rs_adam_variant", "zb_wait_flags", "zb_peer_pull",
                          "zb_ag_gemm_bf16", "zb_gemm2_rs_bf16", "zb_gemm2_rs_bf16", "zb_rs_finish", "zb_tp_norm_push",
                          "zb_tp_norm_push", "zb_tp_push"]
    # argument counts match the C signatures (a miscount would shift every later argument)
    want = {"zb_rs_adam": 23, "zb_rs_adam_nvls": 24, "zb_wait_flags": 7, "zb_peer_pull": 5, "zb_gemm2_rs_bf16": 18,
            "zb_rs_finish": 15, "zb_tp_norm_push": 26, "zb_tp_push": 10}
    for name, nargs in lib.calls:
        if name in want:
            assert nargs == want[name], (name, nargs)


@pytest.mark.parametrize("model,overrides", [("tiny_llama", {}), ("toygpt", {}), ("deepspeedmistral_toy", {}),
                                              ("deepspeedbert_110m", {"layers": 2, "hidden": 128, "heads": 4, "kv_heads": 4, "ffn": 256}),
                                              ("opt_1b", {"layers": 2, "hidden": 128, "heads": 4, "kv_heads": 4, "ffn": 256}),
                                              ("deepspeedvit_default", {"layers": 2, "hidden": 128, "heads": 4, "kv_heads": 4,
                                                                        "ffn": 256, "image": 64, "patch": 16})])
def test_a_whole_step_through_the_gpu_op_layer(lib, model, overrides):
    """One training step per schedule family with the sm100 op layer on top of the stand-in library: every
    call the GPU path would make is made (outputs are meaningless), so a wrong argument, shape or name in the
    layers, the op layer or the wrappers shows up without a GPU; the fixture checks the argument counts."""
    from zorse_b200.config.training_config import parse_pipeline_dict
    from zorse_b200.trainer import Trainer, TrainerOptions

    L = overrides.get("layers", 4)
    cfg = parse_pipeline_dict({"model_name": model, "global_batch_size": 4, "microbatch_size": 2, "sequence_length": 128,
                               "vocab_size": 512, "autocast_dtype": "bfloat16", "reduce_dtype": "bfloat16",
                               "pipeline_config": [{"gpu_ranks": [0], "num_microbatches_per_rank": [2],
                                                    "layer_partition": [0, L], "zero_config": [[0]]}]})
    for schedule, recompute, oib in (("1f1b", False, False), ("zero2", True, True), ("layer_major", None, False)):
        before = len(lib.calls)
        tr = Trainer(cfg, TrainerOptions(schedule=schedule, ops="sm100", activation_recompute=recompute,
                                         optimizer_in_backward=oib, model_overrides=overrides))
        tr.train_step_from_host(tr.synthetic_batch())
        made = {n for n, _ in lib.calls[before:]}
        need = {"zb_norm_fwd", "zb_cross_entropy", "zb_adam"}
        if "vit" not in model:
            need |= {"zb_embedding_fwd", "zb_embedding_bwd"}
        assert need <= made and ({"zb_gemm2_bf16", "zb_gemm_bf16"} & made), sorted(made)
        # whichever version the defaults pick for this shape
        assert {"zb_flash_fwd", "zb_flash_fwd4"} & made and {"zb_flash_bwd", "zb_flash_bwd2", "zb_flash_bwd3"} & made, sorted(made)
        assert {"zb_norm_bwd", "zb_norm_bwd2"} & made, sorted(made)


def test_candidate_report_cases_run_end_to_end_on_the_stand_in_library(lib, monkeypatch):
    """Every case of the candidate report, executed on CPU tensors against the stand-in library (small shapes):
    the tool's own code must not be what fails on the first GPU run."""
    from zorse_b200.profiler import candidates as C

    monkeypatch.setattr(C, "ATTN_SHAPES", {"7b": (1, 256, 4, 4, 128, 0), "gqa64": (2, 128, 4, 2, 64, 0),
                                           "ragged_window": (1, 200, 4, 2, 128, 64)})
    monkeypatch.setattr(C, "NORM_SHAPES", {"7b": (64, 256), "gqa64": (64, 128), "ragged_window": (50, 320)})
    monkeypatch.setattr(C, "WGRAD_SHAPES", {"7b_qkv": (256, 512, 256), "7b_gate_up": (256, 768, 256), "ragged": (100, 300, 264)})
    for case in C.CASES:
        r = C.run_case(case, dev="cpu", flush_floats=16)
        assert r["case"] == case and "max_diff" in r and "tolerance" in r and "agrees" in r, r
        assert "ms_default" in r and "ms_candidate" in r, r          # status word stayed 0 on the stand-in
    table = C.format_table([C.run_case(c, dev="cpu", flush_floats=16) for c in C.CASES[:2]])
    assert table.count("\n") == 3


@pytest.mark.parametrize("kernel", ["fwd4", "bwd2"])
def test_attention_trace_tool_runs_and_copes_with_an_empty_trace(lib, monkeypatch, capsys, tmp_path, kernel):
    """The trace tool end to end on the stand-in library: nothing is recorded (all-zero buffer), which is
    also what a kernel that returned early would leave; the tool must report that instead of failing."""
    from zorse_b200.profiler import attn_trace

    monkeypatch.setattr(k, "check_status", lambda device=None: None)
    out = tmp_path / "trace.json"
    attn_trace.main(["--kernel", kernel, "--S", "256", "--heads", "2", "--kv_heads", "2", "--D", "64", "--ctas", "2",
                     "--device", "cpu", "--out", str(out)])
    assert out.exists() and capsys.readouterr().out.strip()


def test_a_whole_step_with_every_candidate_version_selected(lib, monkeypatch):
    """The same dry run with the opt-in kernel versions selected the way their environment switches do:
    flipping a default must not be what breaks the Python side."""
    from zorse_b200.config.training_config import parse_pipeline_dict
    from zorse_b200.trainer import Trainer, TrainerOptions

    monkeypatch.setattr(k, "ATTN_FWD_VERSION", 4)
    monkeypatch.setattr(k, "ATTN_FWD4_FLAGS", 2)
    monkeypatch.setattr(k, "ATTN_BWD_VERSION", 2)
    monkeypatch.setattr(k, "NORM_FWD_VERSION", 2)
    monkeypatch.setattr(k, "NORM_BWD_VERSION", 2)
    monkeypatch.setattr(k, "GEMM_ACC_PREFETCH", True)
    cfg = parse_pipeline_dict({"model_name": "tiny_llama", "global_batch_size": 4, "microbatch_size": 2,
                               "sequence_length": 256, "vocab_size": 512, "autocast_dtype": "bfloat16",
                               "reduce_dtype": "bfloat16",
                               "pipeline_config": [{"gpu_ranks": [0], "num_microbatches_per_rank": [2],
                                                    "layer_partition": [0, 4], "zero_config": [[0]]}]})
    tr = Trainer(cfg, TrainerOptions(schedule="1f1b", ops="sm100", activation_recompute=False))
    tr.train_step_from_host(tr.synthetic_batch())
    made = {n for n, _ in lib.calls}
    assert {"zb_flash_fwd4", "zb_flash_bwd2", "zb_norm_fwd2", "zb_norm_bwd2", "zb_gemm2_accpf_bf16"} <= made, sorted(made)
    assert not ({"zb_flash_fwd", "zb_flash_bwd", "zb_norm_fwd", "zb_norm_bwd"} & made), sorted(made)


def test_kernel_bench_with_candidate_rows_runs_end_to_end(lib, monkeypatch, tmp_path, capsys):
    """The timing tool, candidate rows included, on the stand-in library with small shapes."""
    from zorse_b200.profiler import kernel_bench as KB

    monkeypatch.setenv("ZORSE_BENCH_CANDIDATES", "1")
    monkeypatch.setattr(KB, "DEV", "cpu")
    monkeypatch.setattr(KB, "_flush", None)
    monkeypatch.setattr(KB, "FLUSH_BYTES", 1024)
    monkeypatch.setattr(KB, "GEMM_SHAPES", [("small", 256, 384, 128)])
    monkeypatch.setattr(KB, "ATTN_CASES", [("small", 1, 256, 4, 2, 64, 0), ("window", 1, 256, 4, 2, 64, 64)])
    monkeypatch.setattr(KB, "ELEMENTWISE_DIMS", (64, 256, 512, 1000, 4096))
    monkeypatch.setattr(k, "check_status", lambda device=None: None)
    out = tmp_path / "kb.json"
    KB.main(["--out", str(out)])
    import json

    rows = json.loads(out.read_text())["rows"]
    ops_seen = {r["op"] for r in rows}
    assert {"gemm wgrad+= 2cta_accpf", "flash fwd v4 mode2", "flash bwd v2", "rmsnorm fwd v2", "rmsnorm bwd v2",
            "gemm fwd 2cta", "flash fwd", "adam (bf16 grad)"} <= ops_seen, sorted(ops_seen)
    assert capsys.readouterr().out.count("\n") == len(rows)


def test_bench_main_prints_its_json_line(lib, monkeypatch, capsys):
    """bench.py from argument parsing to the JSON line, one process, on the stand-in library with stand-in CUDA
    events: every key the benchmark contract names is there."""
    import importlib.util
    import json
    import os
    import sys

    class Ev:
        def __init__(self, enable_timing=False):
            pass

        def record(self, stream=None):
            pass

        def query(self):
            return True

        def elapsed_time(self, other):
            return 12.5

        def synchronize(self):
            pass

    monkeypatch.setattr(k, "check_status", lambda device=None: None)
    monkeypatch.setattr(torch.cuda, "Event", Ev)
    monkeypatch.setattr(torch.cuda, "max_memory_allocated", lambda *a: 0)
    monkeypatch.setattr(torch.cuda, "synchronize", lambda *a: None)
    for var in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_ADDR"):
        monkeypatch.delenv(var, raising=False)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("bench_script", os.path.join(root, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    monkeypatch.setattr(sys, "argv", ["bench.py", "--steps", "2", "--warmup", "3", "--model", "tiny_llama", "--vocab", "512",
                                      "--seq_len", "128", "--global_batch", "4", "--microbatch", "2"])
    assert mod.main() == 0
    line = [ln for ln in capsys.readouterr().out.splitlines() if ln.startswith("{")][-1]
    out = json.loads(line)
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "clocks", "e2e", "gpu_launches"):
        assert key in out, key
    assert out["n_gpus"] == 1 and out["steps"] == 2 and out["warmup"] == 3 and out["ms_per_step"] == 6.25
    assert out["value"] == pytest.approx(4 * 128 / 6.25e-3) and out["gpu_launches"] > 0
    assert {"value", "unit", "h2d_bytes_per_step", "d2h_bytes_per_step"} <= set(out["e2e"])
    assert out["e2e"]["h2d_bytes_per_step"] == 2 * 4 * 128 * 8 and out["e2e"]["d2h_bytes_per_step"] == 4
    assert {"model", "global_batch", "seq_len", "parallelism"} <= set(out["config"])
