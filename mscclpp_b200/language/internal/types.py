"""Import path kept for code written against the reference (`mscclpp.language.internal.types`)."""
from ..types import (BufferType, ChannelType, Chunk, Instruction, RankGroup, ReduceOperationType,  # noqa: F401
                     ReplicationPolicy, SyncType)
