"""supersonic_b200: a small, whole generation library for one B200.

``load(model_dir)`` gives an :class:`Engine`; ``Engine.generate(prompts, ...)`` returns
token ids.  Everything below runs hand-written CUDA for sm_100a; there is no CPU path.
"""
__version__ = "0.1.0"


def load(*args, **kwargs):
    from .api import load as _load
    return _load(*args, **kwargs)


def __getattr__(name):
    if name == "Engine":
        from .api import Engine
        return Engine
    raise AttributeError(name)
