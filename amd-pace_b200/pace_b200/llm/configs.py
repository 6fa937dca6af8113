"""The few configuration records the generation loop needs (reference: pace/llm/configs.py)."""
from dataclasses import dataclass
from typing import Optional


@dataclass
class SamplingConfig:
    """Greedy decoding up to ``max_new_tokens`` (the reference's SamplingConfig reduced to what the
    BASELINE configs use; pace/llm/configs.py:37-432)."""
    max_new_tokens: int = 20
    pad_token_id: int = 0
    eos_token_id: Optional[int] = None
    num_beams: int = 1          # > 1: beam search (generator.py:517-636), the cache follows the beams by index


@dataclass
class PardSpecDecodeConfig:
    """PARD speculative decoding (reference pace/llm/configs.py:529-567): ``num_speculative_tokens``
    draft tokens per step from one parallel draft pass fed with ``pard_token`` placeholders."""
    num_speculative_tokens: int = 12
    pard_token: int = 1
    # batched serving extension: seeded Bernoulli acceptance instead of comparing tokens
    forced_accept_prob: Optional[float] = None
    forced_accept_seed: int = 0
