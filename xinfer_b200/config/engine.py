"""Engine options, named as the reference names them where it has them
(src/utils/config.rs:422-492 and the Python constructor in xinfer.pyi:96-138)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

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
    # ---- options of the reference's EngineConfig for what this engine does not build.  They are accepted so
    # that a script written for the reference constructs its configuration unchanged; a value that asks for the
    # feature is refused by validate() with the feature's name, a value that switches it off is ignored. ----
    device_ids: Optional[List[int]] = None        # one GPU: [i] selects cuda:i
    weight_file: Optional[str] = None             # GGUF files
    isq: Optional[str] = None                     # in-situ quantization
    kvcache_dtype: Optional[str] = None           # quantized caches ("auto" / None: the engine's dtype)
    num_shards: Optional[int] = 1                 # tensor parallelism
    num_nodes: int = 1
    server_mode: Optional[bool] = None
    cpu_mem_fold: Optional[float] = None          # cache pages swapped to host memory
    disable_prefix_cache: bool = False            # there is no prefix cache to disable
    prefix_cache_max_tokens: Optional[int] = None
    disable_reasoning: bool = False               # chat templates are outside this engine
    mtp_num_speculative_tokens: Optional[int] = None
    hf_token: Optional[str] = None
    hf_token_path: Optional[str] = None

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
        not_built = []
        if self.weight_file:
            not_built.append("weight_file (GGUF weights)")
        if self.isq:
            not_built.append("isq (quantized weights)")
        if self.kvcache_dtype not in (None, "", "auto"):
            not_built.append("kvcache_dtype (quantized caches)")
        if self.num_shards not in (None, 1) or self.num_nodes != 1:
            not_built.append("num_shards / num_nodes (more than one GPU)")
        if self.device_ids is not None and len(self.device_ids) != 1:
            not_built.append("device_ids with more than one GPU")
        if self.server_mode:
            not_built.append("server_mode")
        if self.cpu_mem_fold:
            not_built.append("cpu_mem_fold (cache pages in host memory)")
        if self.mtp_num_speculative_tokens:
            not_built.append("mtp_num_speculative_tokens (speculative decoding)")
        if not_built:
            raise ValueError("EngineConfig asks for what this engine does not build: " + "; ".join(not_built))
        if self.device_ids is not None:
            self.device = f"cuda:{int(self.device_ids[0])}"
