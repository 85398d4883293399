from .partition import partition_layers, partition_uniform, partition_balanced  # noqa


def __getattr__(name):
    if name in ("PipelineEngine", "initialize"):
        from . import pipeline
        return getattr(pipeline, name)
    raise AttributeError(name)
