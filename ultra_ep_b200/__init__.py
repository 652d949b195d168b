"""B200-native per-layer expert-balancing hot path behind the ultra_ep.Manager surface.

    from ultra_ep_b200 import Manager, init_runtime, EventHandle

The native parts (ultra_ep_b200/lib/libuep_b200.so and the `_C` extension) are built in-tree by
`python -m ultra_ep_b200.build`. There is no CPU or non-CUDA implementation: importing the
hot-path classes without the built extension raises.
"""

__version__ = "0.1.0"
__all__ = ["Manager", "init_runtime", "EventHandle"]


def __getattr__(name):
    if name == "Manager":
        from .manager import Manager

        return Manager
    if name == "init_runtime":
        from .runtime import init_runtime

        return init_runtime
    if name == "EventHandle":
        from .event import EventHandle

        return EventHandle
    raise AttributeError(f"module 'ultra_ep_b200' has no attribute {name!r}")
