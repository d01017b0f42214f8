"""Engine options, named as the reference names them where it has them
(src/utils/config.rs:422-492 and the Python constructor in xinfer.pyi:96-138)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from .generation import GenerationConfig


@dataclass
class EngineConfig:
    # where the model is: a folder with config.json and model.safetensors
    weight_path: Optional[str] = None
    # alias of weight_path (the reference's `--m`)
    model_id: Optional[str] = None
    # tokens per cache page (`block_size` in the reference, 64 there on CUDA, config.rs:694)
    block_size: int = 16
    # pages per cache group; None = sized from free memory x kv_fraction
    num_blocks: Optional[int] = None
    kv_fraction: float = 0.7
    # most requests alive at once (also the number of per-request state slots)
    max_num_seqs: int = 32
    # most tokens run in one step (prompt portions plus decoded tokens)
    max_num_batched_tokens: int = 8192
    # longest prompt portion of one request in one step
    prefill_chunk_size: int = 8192
    max_model_len: Optional[int] = None
    # default for SamplingParams.max_tokens
    max_tokens: Optional[int] = None
    seed: Optional[int] = None
    # defaults for the sampling options a request leaves unset; they come before those of the model folder's
    # generation_config.json, field by field (the reference's `generation_cfg`)
    generation_cfg: Optional[GenerationConfig] = None
    disable_cuda_graph: bool = False
    # decide and queue the next decode step while the current one runs (the device then does not
    # wait for the host between steps); off: every step waits for its tokens before the next is decided
    disable_run_ahead: bool = False
    device: str = "cuda:0"
    # debug: fill every page that goes back to its pool with NaN before the next step runs
    poison_freed_pages: bool = False

    def model_dir(self) -> str:
        path = self.weight_path or self.model_id
        if not path:
            raise ValueError("EngineConfig needs weight_path (or model_id): a folder with config.json and model.safetensors")
        return path

    def validate(self) -> None:
        for name in ("block_size", "max_num_seqs", "max_num_batched_tokens", "prefill_chunk_size"):
            v = getattr(self, name)
            if not isinstance(v, int) or v <= 0:
                raise ValueError(f"EngineConfig.{name} must be a positive integer, got {v!r}")
        if self.num_blocks is not None and self.num_blocks <= 0:
            raise ValueError(f"EngineConfig.num_blocks must be positive, got {self.num_blocks}")
        if not (0.0 < self.kv_fraction <= 1.0):
            raise ValueError(f"EngineConfig.kv_fraction must lie in (0, 1], got {self.kv_fraction}")
