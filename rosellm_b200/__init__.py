"""rosellm_b200: a single-GPU inference engine for NVIDIA B200 (sm_100a).

``config``    typed configurations and the architecture registry
``weights``   safetensors by tensor name; random-weights mode
``parts``     mixers, feed-forwards, norms, position encodings, blocks
``models``    a model as a list of parts; the GPT-2 builder
``cache``     pages, block tables, per-request state slots
``engine``    the step function, the scheduler, ``LLM``
``sampling``  sampling parameters and the sampler
``ops``       the CUDA library (``csrc``) and its checked Python faces
"""
from . import config, parts  # noqa: F401
from .parts import standard as _standard_parts  # noqa: F401  (registers the shipped parts)
from . import models  # noqa: F401  (registers the shipped architectures)

__version__ = "0.1.0"


def __getattr__(name: str):
    if name in ("LLM", "SamplingParams", "RequestOutput"):
        from .engine import llm

        return getattr(llm, name)
    raise AttributeError(name)
