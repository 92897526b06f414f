"""inferx_b200: a small, whole Qwen2-MoE inference engine for one B200.

    from inferx_b200 import Engine, EngineConfig, Request, SamplingParams
    engine = Engine.create(EngineConfig(model="/path/to/folder", dtype="bfloat16"))
    out = engine.generate([Request([1, 2, 3], SamplingParams(max_tokens=8))])
"""
__version__ = "0.1.0"


def __getattr__(name):
    # heavy imports (torch) only when the public names are first used
    if name in ("Engine", "EngineConfig", "Request"):
        from .engine import engine as _e
        return getattr(_e, name)
    if name == "SamplingParams":
        from .sampling.params import SamplingParams
        return SamplingParams
    if name in ("Completion", "TokenDelta", "TokenLogprob"):
        from .engine import scheduler as _s
        return getattr(_s, name)
    raise AttributeError(name)
