from .hooks import build_hooks, Hook, ComposeHook  # noqa


def __getattr__(name):
    if name in ("BaseRunner",):
        from . import base_llm_runner
        return getattr(base_llm_runner, name)
    if name in ("HFRunner",):
        from . import hf_runner
        return getattr(hf_runner, name)
    raise AttributeError(name)
