"""disagmoe_b200: a Blackwell-native disaggregated MoE serving engine.

Attention layers and expert (FFN) layers run on separate GPU groups; tokens flow layer by layer between them.
Sub-packages: ``config`` (model / cache / sampling dataclasses), ``utils.placement`` (who runs which layer),
``models`` (fp32 oracle, attention and expert modules, weight layout), ``ops`` (sm_100a kernels),
``parallel`` (peer-memory data plane, fused dispatch / combine, tensor parallel collectives),
``frontend`` (controller, engines), ``executor``, ``scheduler`` and the native runtime ``disagmoe_c``.
"""
__version__ = "0.1.0"


def _load_runtime_variant():
    """DMOE_RUNTIME_VARIANT=address|thread: use the sanitizer-instrumented build of the native runtime
    (``build.build_runtime(sanitize=...)``) as ``disagmoe_b200.disagmoe_c``. The process must have the matching
    sanitizer runtime preloaded (``build.sanitizer_runtime``)."""
    import importlib.machinery
    import importlib.util
    import os
    import sys
    import sysconfig
    kind = os.environ.get("DMOE_RUNTIME_VARIANT")
    if not kind:
        return
    import torch  # noqa: F401  (the extension links against libtorch)
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_variants", kind, "disagmoe_c" + suffix)
    loader = importlib.machinery.ExtensionFileLoader("disagmoe_b200.disagmoe_c", path)
    spec = importlib.util.spec_from_loader("disagmoe_b200.disagmoe_c", loader, origin=path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules["disagmoe_b200.disagmoe_c"] = mod
    loader.exec_module(mod)
    globals()["disagmoe_c"] = mod


_load_runtime_variant()
