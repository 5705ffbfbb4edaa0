"""Parts a decoder is put together from.  Importing the package registers the built-in kinds."""
from . import attention, block, combine, latent, mlp, moe, norm, recurrent, rope  # noqa: F401  (registration)
from .base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, Block, BuildEnv, CompositeNeed, FeedForward,
                   KVCacheNeed, KVView, LatentCacheNeed, LayerContext, Mixer, Norm, ParamSpec, Part, PositionEncoding, StateNeed)
from .spec import (AttentionSpec, BlockSpec, ChannelDeltaSpec, ClampedGLUSpec, DecoderSpec, LatentAttentionSpec,
                   MatrixMemorySpec, MixerSumSpec, MoESpec, NormSpec, ParallelBlockSpec, RampedRopeSpec, RetentionSpec,
                   RopeSpec, SandwichBlockSpec, ScaledRopeSpec, ScheduleEntry, SwiGLUSpec)
