"""scratch_llm_b200: a small, whole inference engine for one B200 (sm_100a), for the dense
Llama-style GQA decoder of andreidhoang/scratch_llm.

config/    typed configurations and the architecture registry
weights/   safetensors by tensor name; seeded random weights
parts/     mixer, feed-forward, norm, position encoding, block
cache/     pages, block tables, state slots
engine/    model, step function, scheduler, Python entry point
sampling/  greedy, temperature and nucleus sampling
kernels/   bindings of the CUDA sources in csrc/
"""

__version__ = "0.1.0"

from .engine import (LLM, Request, ServeResult, batched_greedy_decode, generate,  # noqa: E402
                     generate_with_logprobs, serve_continuous, serve_static_wave)
from .sampling import SamplingParams  # noqa: E402

__all__ = ["LLM", "Request", "SamplingParams", "ServeResult", "batched_greedy_decode",
           "generate", "generate_with_logprobs", "serve_continuous", "serve_static_wave"]
