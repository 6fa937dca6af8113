"""Output records of the model and the generator (reference: pace/llm/outputs.py)."""
from dataclasses import dataclass
from typing import List, Optional

import torch


@dataclass
class ModelOutput:
    logits: torch.Tensor


@dataclass
class SpeculativeStats:
    total_speculated_tokens: int
    mean_accepted_tokens: float


@dataclass
class GeneratorOutput:
    output_token_ids: torch.Tensor                 # [B, longest]; shorter rows padded with pad_token_id
    lengths: List[int]                             # tokens per row (prompt included)
    speculative_stats: Optional[SpeculativeStats] = None
