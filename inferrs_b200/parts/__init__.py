"""Parts that models are assembled from; importing the package registers the built-in ones."""
from . import attention, basic, blocks, combine, feed_forward, latent_attention, recurrent  # noqa: F401
from .registry import (PartError, part_class, register_arrangement, register_feed_forward, register_mixer,
                       register_norm, register_part, register_position)
from .spec import (AttentionSpec, ChannelDecayScanSpec, FixedDecayScanSpec, ForgetWriteScanSpec, InputConvSpec, GatedDeltaScanSpec, GatedDenseSpec,
                   MixerSumSpec, ResidualGateSpec, RoutedExpertsSpec,
                   StateSpaceScanSpec, LatentAttentionSpec, LayerSpec, ModelSpec,
                   NormSpec, PolyNormDenseSpec, PositionSpec, ScalarGateScanSpec, ScheduleEntry, StreamConnectionSpec,
                   SubLayerSpec, TensorDecl, default_schedule, pre_norm_layer)
