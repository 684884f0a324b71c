"""Model zoo: name -> architecture -> list of layers (the units the engine shards).

Covers the families of the reference registry (models/hub.py:25-84, 535-671): Llama in
both of its styles (`deepspeedllama_*`, `deepspeedllamav2_*`), Mistral, GPT
(`deepspeedgpt_*`, `toygpt*`), OPT, BERT and ViT, under the same names, plus the models
the benchmark configurations name (`llama3.2_1b`, `llama2_7b`, `mistral_7b`, `opt_13b`,
`tiny_llama`) and the names of the reference's HF whole-model wrappers (`llama_*`, `gpt_*`,
`bert_*`, `vit_*`, `opt_*`, `mistral_*`; models/llama.py, gpt.py, bert.py, vit.py, opt.py, mistral.py).  Unlike the reference every family here can be split into pipeline stages:
`build_stage_layers` returns `[embedding?] + blocks[start:end] + [head?]`.
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Optional

from .layers import EmbeddingLayer, HeadLayer, Layer, NoOpLayer, PatchEmbeddingLayer, TransformerBlock


@dataclass(frozen=True)
class ModelSpec:
    name: str
    family: str            # llama | mistral | gpt | opt | bert | vit
    layers: int
    hidden: int
    heads: int
    ffn: int
    kv_heads: Optional[int] = None
    vocab: int = 32000
    norm: str = "rms"
    pre_norm: bool = True
    act: str = "swiglu"
    bias: bool = False
    rope_theta: Optional[float] = 10000.0
    causal: bool = True
    window: int = 0
    max_positions: int = 0
    pos_offset: int = 0
    eps: float = 1e-5
    embed_norm: bool = False
    head_norm: Optional[str] = "rms"
    pool: Optional[str] = None
    image: int = 0
    patch: int = 0
    classes: int = 0
    init_std: float = 0.02

    @property
    def head_dim(self) -> int:
        return self.hidden // self.heads

    @property
    def n_kv(self) -> int:
        return self.kv_heads or self.heads


def _llama(name, L, H, heads, F, **kw):
    return ModelSpec(name, "llama", L, H, heads, F, **kw)


def _gpt(name, L, H, heads, **kw):
    d = dict(norm="ln", act="gelu", bias=True, rope_theta=None, max_positions=2048, head_norm="ln", vocab=50257)
    d.update(kw)
    return ModelSpec(name, d.pop("family", "gpt"), L, H, heads, d.pop("ffn", 4 * H), **d)


def _opt(name, L, H, heads):
    # OPT: pre-LN, learned positions with an offset of 2, ReLU in the released checkpoints;
    # the benchmark configuration asks for GELU, selectable with act= at build time.
    return _gpt(name, L, H, heads, family="opt", act="gelu", vocab=50272, max_positions=2048, pos_offset=2)


def _bert(name, L, H, heads):
    return ModelSpec(name, "bert", L, H, heads, 4 * H, vocab=30522, norm="ln", pre_norm=False, act="gelu_erf", bias=True,
                     rope_theta=None, causal=True, max_positions=512, embed_norm=True, head_norm=None, eps=1e-12)


def _vit(name, L, H, heads, F):
    return ModelSpec(name, "vit", L, H, heads, F, vocab=0, norm="ln", pre_norm=True, act="gelu_erf", bias=True,
                     rope_theta=None, causal=False, head_norm="ln", pool="first", image=384, patch=16, classes=10,
                     eps=1e-12)


_SPECS: dict[str, ModelSpec] = {}


def _reg(spec: ModelSpec):
    _SPECS[spec.name] = spec


for _style in ("deepspeedllama", "deepspeedllamav2"):
    _reg(_llama(f"{_style}_tiny", 22, 2048, 32, 5632))
    _reg(_llama(f"{_style}_3b", 26, 3200, 32, 8640))
    _reg(_llama(f"{_style}_7b", 32, 4096, 32, 11008))
    _reg(_llama(f"{_style}_13b", 40, 5120, 40, 13824))
    _reg(_llama(f"{_style}_33b", 60, 6656, 52, 17920))
    _reg(_llama(f"{_style}_65b", 80, 8192, 64, 22016))
_reg(_llama("llama2_7b", 32, 4096, 32, 11008))
_reg(_llama("llama3.2_1b", 16, 2048, 32, 8192, kv_heads=8, vocab=128256, rope_theta=500000.0))
_reg(_llama("tiny_llama", 4, 512, 8, 1376, vocab=32000))
_reg(replace(_llama("deepspeedmistral_7b", 32, 4096, 32, 14336, kv_heads=8, window=4096), family="mistral"))
_reg(replace(_llama("mistral_7b", 32, 4096, 32, 14336, kv_heads=8, window=4096), family="mistral"))
_reg(replace(_llama("deepspeedmistral_toy", 4, 512, 8, 1376, kv_heads=2, window=64), family="mistral"))

_reg(_gpt("deepspeedgpt_test", 12, 512, 8))
_reg(_gpt("deepspeedgpt_1.3b", 24, 2048, 16))
_reg(_gpt("deepspeedgpt_2.7b", 32, 2560, 20))
_reg(_gpt("deepspeedgpt_6.7b", 32, 4096, 32))
_reg(_gpt("deepspeedgpt_13b", 40, 5120, 40))
_reg(_gpt("deepspeedgpt_175b", 96, 12288, 96))
_reg(_gpt("toygpt", 4, 256, 4, vocab=1024, max_positions=256))
_reg(_gpt("toygpt_small", 2, 128, 2, vocab=512, max_positions=128))

for _n, (_L, _H, _h) in {"125m": (12, 768, 12), "350m": (24, 1024, 16), "1b": (24, 2048, 32), "2b": (24, 2560, 32),
                          "3b": (32, 2560, 32), "4b": (24, 3648, 32), "5b": (24, 4096, 32), "6.7b": (32, 4096, 32),
                          "13b": (40, 5120, 40), "30b": (48, 7168, 56), "66b": (64, 9216, 72),
                          "175b": (96, 12288, 96)}.items():
    _reg(_opt(f"opt_{_n}", _L, _H, _h))

for _n, (_L, _H, _h) in {"110m": (12, 768, 12), "base": (12, 768, 12), "330m": (24, 1024, 16), "large": (24, 1024, 16),
                          "1b": (24, 1824, 32), "2b": (24, 2560, 32), "3b": (24, 3172, 32), "4b": (24, 3648, 32),
                          "5b": (24, 4096, 32), "xlarge": (36, 1536, 24)}.items():
    _reg(_bert(f"deepspeedbert_{_n}", _L, _H, _h))

for _n, (_L, _H, _h, _F) in {"default": (12, 768, 12, 3072), "1b": (24, 1824, 32, 7296), "2b": (24, 2560, 32, 10240),
                              "3b": (24, 3172, 32, 12688), "4b": (24, 3648, 32, 14592), "5b": (24, 4096, 32, 16384),
                              "h": (32, 1280, 16, 5120), "g_small": (6, 1664, 16, 8192), "g": (48, 1664, 16, 8192),
                              "e_small": (6, 1792, 16, 15360), "e": (56, 1792, 16, 15360)}.items():
    _reg(_vit(f"deepspeedvit_{_n}", _L, _H, _h, _F))


# ---- names of the reference's whole-model wrappers (models/llama.py, gpt.py, bert.py, vit.py,
# mistral.py): HF-config models at named sizes that the reference can only profile or run on a
# single stage.  Same dimensions here, and like every other entry they can be pipelined.
for _n, (_L, _H, _h) in {"1b": (24, 1536, 32), "2b": (24, 2176, 32), "3b": (24, 2688, 32), "4b": (24, 3136, 32),
                          "5b": (24, 3520, 32), "6.7b": (32, 4096, 32), "13b": (40, 5120, 40), "33b": (60, 6656, 52),
                          "65b": (80, 8192, 64)}.items():
    _reg(_llama(f"llama_{_n}", _L, _H, _h, 4 * _H, vocab=49152))      # FFN = 4 x hidden (models/llama.py:49-50)
for _n, (_L, _H, _h) in {"85m": (12, 768, 12), "300m": (24, 1024, 16), "1b": (24, 1824, 32), "1b_1l": (1, 1824, 32),
                          "1.3b": (24, 2048, 128), "2b": (24, 2560, 32), "2.7b": (32, 2560, 80), "3b": (24, 3328, 32),
                          "4b": (24, 3648, 32), "5b": (24, 4096, 32), "6b": (32, 4096, 32), "6.7b": (32, 4096, 128),
                          "10b": (36, 4680, 36), "20b": (44, 6144, 48), "25b": (46, 6656, 52), "30b": (48, 7168, 56),
                          "35b": (53, 7424, 58), "40b": (54, 7808, 61), "45b": (56, 8192, 64), "50b": (58, 8448, 66),
                          "55b": (61, 8704, 68), "60b": (62, 8960, 70), "65b": (64, 9216, 72)}.items():
    # OpenAI-GPT style (post-LN); `gpt_13b` of the reference (5140 / 128 heads) is not a valid shape and is left out
    _reg(_gpt(f"gpt_{_n}", _L, _H, _h, pre_norm=False, vocab=49152))
for _n, (_L, _H, _h, _F) in {"110m": (12, 768, 12, 0), "330m": (24, 1024, 16, 0), "1b": (24, 1824, 32, 0),
                              "2b": (24, 2560, 32, 0), "3b": (24, 3172, 32, 0), "4b": (24, 3648, 32, 0),
                              "5b": (24, 4096, 32, 0), "large": (24, 1024, 16, 4096), "xlarge": (36, 1536, 24, 6144)}.items():
    _reg(replace(_bert(f"bert_{_n}", _L, _H, _h), ffn=_F or 4 * _H, vocab=49152))
for _n, (_L, _H, _h, _F) in {"default": (12, 768, 12, 0), "1b": (24, 1824, 32, 0), "2b": (24, 2560, 32, 0),
                              "3b": (24, 3172, 32, 0), "4b": (24, 3648, 32, 0), "5b": (24, 4096, 32, 0),
                              "g": (48, 1664, 16, 8192), "e": (56, 1792, 16, 15360)}.items():
    _reg(replace(_vit(f"vit_{_n}", _L, _H, _h, _F or 4 * _H), image=224, classes=2))   # HF ViTConfig defaults
_reg(replace(_llama("mistral_toy", 5, 4096, 32, 14336, kv_heads=8, window=4096, vocab=49152), family="mistral"))


def list_models() -> list[str]:
    return sorted(_SPECS)


def get_spec(name: str, **overrides) -> ModelSpec:
    """Architecture of a registered model; keyword overrides (layers=, vocab=, act=, ...)
    replace fields, as the reference does with `layers=` / `vocab_size=` kwargs."""
    if name not in _SPECS:
        raise ValueError(f"Unsupported model: {name}. Known: {', '.join(list_models())}")
    spec = _SPECS[name]
    ov = {k: v for k, v in overrides.items() if v is not None}
    if "vocab_size" in ov:
        ov["vocab"] = ov.pop("vocab_size")
    if spec.family == "vit":
        ov.pop("vocab", None)
    return replace(spec, **ov) if ov else spec


def get_config_for_model(name: str):
    """(num_transformer_layers, hidden_size, num_attention_heads, intermediate_size)."""
    s = get_spec(name)
    return s.layers, s.hidden, s.heads, s.ffn


def _tp_kw(tp: int, tp_index: int) -> dict:
    return {} if tp == 1 else {"tp": tp, "tp_index": tp_index}


def make_block(spec: ModelSpec, tp: int = 1, tp_index: int = 0) -> TransformerBlock:
    """One transformer block; with tp > 1 slice `tp_index` of it (models/tp_layers.py)."""
    cls = TransformerBlock
    if tp > 1:
        from .tp_layers import TPTransformerBlock as cls
    return cls(spec.hidden, spec.heads, spec.n_kv, spec.ffn, norm=spec.norm, pre_norm=spec.pre_norm,
               act=spec.act, bias=spec.bias, rope_theta=spec.rope_theta, causal=spec.causal,
               window=spec.window, eps=spec.eps, init_std=spec.init_std, **_tp_kw(tp, tp_index))


def make_embedding(spec: ModelSpec, seq_len: int, tp: int = 1, tp_index: int = 0) -> Layer:
    if spec.family == "vit":
        if tp > 1:
            raise NotImplementedError("tensor parallelism does not cover the ViT patch embedding")
        return PatchEmbeddingLayer(spec.image, spec.patch, 3, spec.hidden, spec.init_std)
    maxpos = max(spec.max_positions, seq_len) if spec.max_positions else 0
    cls = EmbeddingLayer
    if tp > 1:
        from .tp_layers import SPEmbeddingLayer as cls
    return cls(spec.vocab, spec.hidden, max_positions=maxpos, pos_offset=spec.pos_offset,
               post_norm=spec.embed_norm, eps=spec.eps, init_std=spec.init_std, **_tp_kw(tp, tp_index))


def make_head(spec: ModelSpec, tp: int = 1, tp_index: int = 0) -> HeadLayer:
    out = spec.classes if spec.family == "vit" else spec.vocab
    cls = HeadLayer
    if tp > 1:
        from .tp_layers import SPHeadLayer as cls
    return cls(spec.hidden, out, norm=spec.head_norm, eps=spec.eps, pool=spec.pool, init_std=spec.init_std,
               **_tp_kw(tp, tp_index))


def build_stage_layers(spec: ModelSpec, layer_start: int, layer_end: int, seq_len: int,
                       insert_noop: bool = False, tp: int = 1, tp_index: int = 0) -> list[Layer]:
    """Layers of the pipeline stage owning blocks [layer_start, layer_end): the first stage
    also owns the embedding, the last one the final norm + head (+ loss).  With tp > 1 the
    layers are this process's tensor-parallel slices."""
    if not (0 <= layer_start < layer_end <= spec.layers):
        raise ValueError(f"bad layer range [{layer_start},{layer_end}) for {spec.name} with {spec.layers} layers")
    out: list[Layer] = []
    if layer_start == 0:
        out.append(make_embedding(spec, seq_len, tp, tp_index))
    out += [make_block(spec, tp, tp_index) for _ in range(layer_start, layer_end)]
    if insert_noop:
        out.append(NoOpLayer())
    if layer_end == spec.layers:
        out.append(make_head(spec, tp, tp_index))
    return out


def global_layer_index(spec: ModelSpec, layer_start: int, local_index: int, layers: list[Layer]) -> int:
    """Stable id of a layer across any stage split (seeds parameter init): embedding = 0,
    block i = 1 + i, head = 1 + L, no-op = 2 + L + position."""
    ly = layers[local_index]
    if ly.kind == "embedding":
        return 0
    if ly.kind == "head":
        return 1 + spec.layers
    if ly.kind == "noop":
        return 2 + spec.layers + local_index
    first_block = 1 if layers[0].kind == "embedding" else 0
    return 1 + layer_start + (local_index - first_block)


# ---- statistics (what data/model_stats.json holds in the reference) -------------------
def params_per_block(spec: ModelSpec) -> int:
    return make_block(spec).num_params()


def total_params(spec: ModelSpec, seq_len: int = 0) -> int:
    return spec.layers * params_per_block(spec) + make_embedding(spec, seq_len).num_params() + make_head(spec).num_params()


def get_model_stats(name: str, **overrides) -> dict:
    s = get_spec(name, **overrides)
    return {"hidden_size": s.hidden, "num_layers": s.layers, "parameters_per_layer": params_per_block(s),
            "total_parameters": total_params(s)}


def write_model_stats(path: str) -> dict:
    """Writes the statistics of every registered model as JSON (the layout of the reference's
    data/model_stats.json: model -> hidden_size, num_layers, parameters_per_layer,
    total_parameters)."""
    import json

    table = {name: get_model_stats(name) for name in list_models()}
    with open(path, "w") as f:
        json.dump(table, f, indent=2)
    return table


if __name__ == "__main__":
    import sys

    out = sys.argv[1] if len(sys.argv) > 1 else "data/model_stats.json"
    print(f"{len(write_model_stats(out))} models -> {out}")
