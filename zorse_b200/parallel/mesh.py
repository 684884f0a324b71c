"""Regular parallel layouts by their four sizes.

`ParallelDims(dp_replicate, dp_shard, tp, pp)` describes a job whose `pp` pipeline stages all have
the same width: `dp_replicate` groups of `dp_shard` ZeRO ranks (more than one group = hybrid
shard), every rank being a lane of `tp` tensor-parallel processes.  `training_config()` writes the
layout as the dictionary the trainer reads (the planner writes the same format for irregular
layouts).  The reference has the four sizes only as an unused device-mesh helper
(utils/parallelism.py:1-104); here they produce a config every schedule can run.

Process numbering: lane `s * dp + g * dp_shard + j` is shard `j` of replicate group `g` of stage
`s`; its processes are `lane * tp .. lane * tp + tp - 1`, so the tensor-parallel processes are
neighbours, then the shard group, then the replicas, then the stages.
"""
from __future__ import annotations

from dataclasses import dataclass

from ..config.training_config import split_evenly


@dataclass
class ParallelDims:
    dp_replicate: int = 1
    dp_shard: int = 1
    tp: int = 1
    pp: int = 1

    def __post_init__(self):
        for k in ("dp_replicate", "dp_shard", "tp", "pp"):
            if getattr(self, k) < 1:
                raise ValueError(f"{k} must be at least 1")

    @property
    def dp(self) -> int:
        return self.dp_replicate * self.dp_shard

    @property
    def world_size(self) -> int:
        return self.dp * self.tp * self.pp

    def lane(self, stage: int, replica: int, shard: int) -> int:
        return stage * self.dp + replica * self.dp_shard + shard

    def processes_of_lane(self, lane: int) -> tuple[int, ...]:
        return tuple(lane * self.tp + t for t in range(self.tp))

    def coordinates(self, process: int) -> dict:
        """Inverse of the numbering: {'pp', 'dp_replicate', 'dp_shard', 'tp'} of a process rank."""
        lane, t = divmod(process, self.tp)
        stage, rest = divmod(lane, self.dp)
        replica, shard = divmod(rest, self.dp_shard)
        return {"pp": stage, "dp_replicate": replica, "dp_shard": shard, "tp": t}

    def training_config(self, model_name: str, num_layers: int, global_batch_size: int, microbatch_size: int,
                        sequence_length: int, zero_level: int = 3, **extra) -> dict:
        if num_layers < self.pp:
            raise ValueError(f"{num_layers} layers cannot fill {self.pp} stages")
        if global_batch_size % microbatch_size:
            raise ValueError("global_batch_size must be a multiple of microbatch_size")
        per_rank = list(split_evenly(global_batch_size // microbatch_size, self.dp))
        cuts = [0]
        for n in split_evenly(num_layers, self.pp):
            cuts.append(cuts[-1] + n)
        stages = []
        for s in range(self.pp):
            groups = [[self.lane(s, g, j) for j in range(self.dp_shard)] for g in range(self.dp_replicate)]
            stages.append({"gpu_ranks": [r for g in groups for r in g], "num_microbatches_per_rank": per_rank,
                           "layer_partition": [cuts[s], cuts[s + 1]], "zero_config": groups,
                           **({"zero_level": zero_level} if zero_level != 3 else {})})
        d = {"model_name": model_name, "global_batch_size": global_batch_size, "microbatch_size": microbatch_size,
             "sequence_length": sequence_length, "pipeline_config": stages}
        if self.tp > 1:
            d["tensor_parallel_size"] = self.tp
        d.update(extra)
        return d


def main(argv=None) -> int:
    """`python -m zorse_b200.parallel.mesh --pp 4 --dp_shard 2 --model_name llama2_7b ...` prints the
    training config of a regular layout (redirect it to a file for `zorse.py --config_file`)."""
    import argparse
    import json

    from ..models import registry

    ap = argparse.ArgumentParser(description=main.__doc__)
    ap.add_argument("--dp_replicate", type=int, default=1)
    ap.add_argument("--dp_shard", type=int, default=1)
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--pp", type=int, default=1)
    ap.add_argument("--model_name", required=True)
    ap.add_argument("--global_batch_size", type=int, required=True)
    ap.add_argument("--microbatch_size", type=int, default=1)
    ap.add_argument("--sequence_length", type=int, required=True)
    ap.add_argument("--vocab_size", type=int, default=None)
    ap.add_argument("--zero_level", type=int, default=3, choices=[2, 3])
    ap.add_argument("--schedule", default=None)
    a = ap.parse_args(argv)
    dims = ParallelDims(a.dp_replicate, a.dp_shard, a.tp, a.pp)
    spec = registry.get_spec(a.model_name, vocab=a.vocab_size)
    extra = {"vocab_size": spec.vocab}
    if a.schedule:
        extra["schedule"] = a.schedule
    d = dims.training_config(a.model_name, spec.layers, a.global_batch_size, a.microbatch_size, a.sequence_length,
                             zero_level=a.zero_level, **extra)
    print(json.dumps(d, indent=1))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
