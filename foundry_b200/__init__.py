"""foundry_b200: a small generation library for the Llama dense decoder on
NVIDIA B200 (sm_100a): from a model folder to generated token ids on one GPU.

    import foundry_b200 as fb
    engine = fb.Engine.from_folder("path/to/model", dtype="bfloat16")
    out = engine.generate([[1, 2, 3], [4, 5]], max_new_tokens=16)
    out.token_ids          # new tokens of each prompt
"""
from .config import LlamaConfig, Llama3RopeScaling, load_model_config
from .engine import Engine, Generation, SequenceStep
from .sampling import SamplingParams
from .weights import write_model_folder

__version__ = "0.1.0"
__all__ = ["LlamaConfig", "Llama3RopeScaling", "load_model_config", "Engine", "Generation",
           "SequenceStep", "SamplingParams", "write_model_folder", "__version__"]
