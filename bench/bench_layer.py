"""python -m bench.bench_layer --seq_length 4096 --profile_batches 4 --autocast_dtype bfloat16 --model_name llama2_7b

Profiles one transformer block on this machine's GPU and rewrites data/model_latencies.json
(reference bench/bench_layer.py, driven by profile_models.sh)."""
import argparse
import json


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--seq_length", type=int, default=4096)
    ap.add_argument("--profile_batches", type=int, default=4)
    ap.add_argument("--autocast_dtype", default="bfloat16")
    ap.add_argument("--reduce_dtype", default="float32")
    ap.add_argument("--model_name", required=True)
    ap.add_argument("--output", default=None, help="latency table to update (default data/model_latencies.json)")
    ap.add_argument("--chain_blocks", type=int, default=4,
                    help="also time this many consecutive blocks against single-block runs and store the ratio (0: skip)")
    a = ap.parse_args(argv)
    from zorse_b200.profiler.layer import profile_and_store

    res = profile_and_store(a.model_name, a.seq_length, a.autocast_dtype, a.profile_batches, a.output,
                            chain_blocks=a.chain_blocks)
    print(json.dumps({"model": a.model_name, "seq": a.seq_length, **res}))


if __name__ == "__main__":
    main()
