"""disagmoe_b200: a Blackwell-native disaggregated MoE serving engine.

Attention layers and expert (FFN) layers run on separate GPU groups; tokens flow layer by layer between them.
Sub-packages: ``config`` (model / cache / sampling dataclasses), ``utils.placement`` (who runs which layer),
``models`` (fp32 oracle, attention and expert modules, weight layout), ``ops`` (sm_100a kernels),
``parallel`` (peer-memory data plane, fused dispatch / combine, tensor parallel collectives),
``frontend`` (controller, engines), ``executor``, ``scheduler`` and the native runtime ``disagmoe_c``.
"""
__version__ = "0.1.0"
