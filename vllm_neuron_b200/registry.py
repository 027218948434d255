"""Model registry: architecture name (config.json) -> how to read its configuration, open its checkpoint and build the
model object the runner steps.

Two families are served:
  * dense Llama / Qwen2 decoders (`B200CausalLM`): HF config.json (`architectures`), HF tensor names; a step is one prefill
    or a batch of decodes;
  * hybrid decoders (`HybridCausalLM`): config.json lists the layers; a step is one ragged batch.  "Pumopel": state-space /
    windowed-attention mixers, Dynamic-Tanh norms, MoE; "Kenetar": delta-rule / latent-attention mixers, post-norm RMS,
    bigram embedding, dense or MoE feed-forward; "Zudarax": parallel mixer / feed-forward branches behind one grouped RMS
    norm, three rotating-attention variants (chunked + soft-capped, differential, sigmoid), polynomial activation;
    "Gerupel": parallel branches behind two RMS norms, a mixer that is windowed attention with pooled far blocks beside a gated
    linear recurrence, repeated layer runs with shared weights, MoE, logits from the embedding table.
The reference resolves the architecture the same way -- `hf_config.architectures[0]` picks the NxDI model class
(vllm_neuron/worker/neuronx_distributed_model_loader.py:612-660).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from types import SimpleNamespace
from typing import Callable

import torch


@dataclass
class ModelEntry:
    family: str                  # "dense" | "hybrid"
    read_config: Callable        # config.json dict -> configuration object
    open_weights: Callable       # (checkpoint dir, configuration) -> weight source
    build: Callable              # (configuration, weights, **engine sizes) -> model
    dtypes: tuple = (torch.bfloat16,)


def _dense_config(d: dict):
    from .config import ModelShape

    return ModelShape.from_hf(SimpleNamespace(**d))


def _dense_weights(path: str, shape, **kw):
    from .loader import HFCheckpointWeights

    return HFCheckpointWeights(path, shape, **kw)


def _dense_build(shape, weights, *, dtype=torch.bfloat16, **kw):
    from .model import B200CausalLM

    if dtype != torch.bfloat16:
        raise ValueError("the dense decoders are served in bfloat16 (optionally with 8-bit weights), not in float32")
    return B200CausalLM(shape, weights, **kw)


def _hybrid_config(d: dict):
    from .hybrid import HybridConfig

    return HybridConfig.from_dict(d)


def _hybrid_weights(path: str, cfg):
    from .loader import CheckpointTensors

    return CheckpointTensors(path)


def _hybrid_build(cfg, weights, *, dtype=torch.bfloat16, **kw):
    from .hybrid import HybridCausalLM

    return HybridCausalLM(cfg, weights, dtype=dtype, **kw)


_DENSE = ModelEntry("dense", _dense_config, _dense_weights, _dense_build)
MODEL_REGISTRY: dict[str, ModelEntry] = {
    "LlamaForCausalLM": _DENSE,
    "Qwen2ForCausalLM": _DENSE,
    "Pumopel": ModelEntry("hybrid", _hybrid_config, _hybrid_weights, _hybrid_build, (torch.bfloat16, torch.float32)),
    "Kenetar": ModelEntry("hybrid", _hybrid_config, _hybrid_weights, _hybrid_build, (torch.bfloat16, torch.float32)),
    "Zudarax": ModelEntry("hybrid", _hybrid_config, _hybrid_weights, _hybrid_build, (torch.bfloat16, torch.float32)),
    "Gerupel": ModelEntry("hybrid", _hybrid_config, _hybrid_weights, _hybrid_build, (torch.bfloat16, torch.float32)),
}


def architecture_of(config: dict) -> str:
    """HF configs name their class under `architectures`; layer-list configs under `architecture`."""
    archs = config.get("architectures")
    return archs[0] if archs else config.get("architecture", "")


def resolve(config: dict) -> tuple[str, ModelEntry]:
    arch = architecture_of(config)
    if arch not in MODEL_REGISTRY:
        raise ValueError(f"architecture {arch!r} is not served (known: {sorted(MODEL_REGISTRY)})")
    return arch, MODEL_REGISTRY[arch]


def load_config(path: str) -> tuple[str, ModelEntry, object]:
    with open(os.path.join(path, "config.json")) as f:
        d = json.load(f)
    arch, entry = resolve(d)
    return arch, entry, entry.read_config(d)
