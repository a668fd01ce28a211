from .sharded import BatchShardedRunner, gather_batch, shard_bounds

__all__ = ["ExecutionEngine", "Torch_ExecutionEngine", "BatchShardedRunner", "gather_batch", "shard_bounds"]


def __getattr__(name):
    # the engines need the llcompiler_ extension (and a GPU); the sharding helpers do not
    if name in ("ExecutionEngine", "Torch_ExecutionEngine", "TORCH_DTYPE_TO_TYPE"):
        from . import engine
        return getattr(engine, name)
    raise AttributeError(name)
