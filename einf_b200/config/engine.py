"""Options of the engine around the model: cache pool, token budget, policy.

Names follow the reference where it has them: ``block_len`` and ``num_blocks``
(``scripts/run_qwen.py:46-47``), ``max_batch_len`` and ``max_prefill_chunk_len``
(``crates/einf-control/src/scheduler.rs:15-18``), the policy strings ``fcfs`` and
``decode_first`` (``crates/einf-control-py/src/lib.rs:663-675``).
"""
from __future__ import annotations

from dataclasses import dataclass

DTYPES = ("bfloat16", "float32")
POLICIES = ("fcfs", "decode_first")


@dataclass(frozen=True)
class EngineConfig:
    dtype: str = "bfloat16"
    block_len: int = 16
    #: pages of every cache group, when ``max_tokens`` is not given
    num_blocks: int = 256
    #: if set, the pool of each group is sized to hold this many tokens
    max_tokens: int | None = None
    max_batch_len: int = 128
    max_prefill_chunk_len: int = 128
    policy: str = "fcfs"
    #: most requests that may hold cache at one time (block-table rows, state slots)
    max_requests: int = 64
    #: most tokens (prompt and generated) one request may reach; None: what the cache pool and the
    #: model's ``max_position_embeddings`` allow.  Block tables are this wide, and a step that is
    #: planned one at a time sends them to the device whole, so a serving limit well below the
    #: model's 32,768 positions spares most of that copy (65 KB -> 8 KB a step at a limit of 4,096).
    max_sequence_len: int | None = None
    #: capture decode-only steps in CUDA graphs
    use_cuda_graphs: bool = True
    #: decode steps the engine may run on the device before it reports to the host, when every
    #: request of a step decodes and none waits (each step's input is then the token sampled in the
    #: step before, fed on the device).  1: every step reports, as the reference does.  With more, a
    #: request that ends on an end-of-sequence token is noticed up to that many steps late (the
    #: surplus tokens are dropped) and a new request waits up to that many steps for admission.
    decode_lookahead: int = 1
    #: with a lookahead: hand every step's tokens to the host (and on to the scheduler and the
    #: caller) as soon as that step is done, while the later steps of the plan run; false: one
    #: report when the whole plan is done
    report_every_step: bool = True
    device: str = "cuda:0"

    def __post_init__(self) -> None:
        if self.dtype not in DTYPES:
            raise ValueError(f"dtype must be one of {DTYPES}, got {self.dtype!r}")
        if self.policy not in POLICIES:
            raise ValueError(f"policy must be one of {POLICIES}, got {self.policy!r}")
        for name in ("block_len", "num_blocks", "max_batch_len", "max_prefill_chunk_len", "max_requests",
                     "decode_lookahead"):
            if getattr(self, name) <= 0:
                raise ValueError(f"{name} must be positive, got {getattr(self, name)!r}")
        if self.max_tokens is not None and self.max_tokens <= 0:
            raise ValueError(f"max_tokens must be positive, got {self.max_tokens!r}")
        if self.max_sequence_len is not None and self.max_sequence_len <= 0:
            raise ValueError(f"max_sequence_len must be positive, got {self.max_sequence_len!r}")
