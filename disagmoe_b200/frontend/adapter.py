"""Names of the native runtime classes for type annotations (reference: disagmoe/frontend/adapter.py).

The native module is :mod:`disagmoe_b200.disagmoe_c`; importing the names from here keeps Python files importable when
the extension has not been built yet (the names are then ``None``)."""
try:
    from ..disagmoe_c import (AttentionBatch, AttentionBatchMetadata, AttentionScheduler, BlockManager, Channel,
                              ChannelInfo, Metadata, MuAttnDispatcher, MuDispatcher, MuExpertDispatcher, MuPool,
                              NcclChannel, NcclGroupChannel, ParallelConfig, Sampler, Scheduler, SloStat, TensorBatch,
                              Tokenizer, TopKSampler)
except ImportError:   # extension not built
    AttentionBatch = AttentionBatchMetadata = AttentionScheduler = BlockManager = Channel = ChannelInfo = Metadata = None
    MuAttnDispatcher = MuDispatcher = MuExpertDispatcher = MuPool = NcclChannel = NcclGroupChannel = ParallelConfig = None
    Sampler = Scheduler = SloStat = TensorBatch = Tokenizer = TopKSampler = None
