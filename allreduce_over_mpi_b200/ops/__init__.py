from .reduce import HostReducePipeline, reduce_nway, reduce_nway_scaled, cpu_reduce, launch_count  # noqa: F401
