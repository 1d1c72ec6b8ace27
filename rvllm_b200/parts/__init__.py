"""Parts a model is put together from: mixers, feed-forwards, norms, position
encodings and their arrangement in a block.  Importing the package registers the
built-in kinds."""
from . import (attention, attention_latent, attention_mixed, block, feed_forward, gated_delta,  # noqa: F401
               hyper, mingru, mlstm, norm, parallel, position, short_conv)
from .base import (Arrangement, FeedForward, Mixer, Norm, PagedNeed, PositionEncoding,
                   SeveralNeeds, StateNeed, Stream, arrangement_class, feed_forward_class, mixer_class,
                   norm_class, position_class, register_arrangement,
                   register_feed_forward, register_mixer, register_norm,
                   register_position)
from .spec import (AttentionSpec, BlockSpec, FeedForwardSpec, LayerCall, MixerSpec,
                   ModelSpec, NormSpec, ParamDecl, PositionSpec, ShortConvSpec, SwiGLUSpec,
                   DenseSpec, MinGRUSpec, MixedAttentionSpec, LatentAttentionSpec, MoESpec,
                   GatedDeltaSpec, GluClampSpec, MLSTMSpec, ParallelSpec)
