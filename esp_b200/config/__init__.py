from .plan import (AttentionSpec, BlockSpec, DecayBonusRecurrenceSpec, DenseFfnSpec, DepthMixBlockSpec,
                   LatentAttentionSpec, LowerBoundRecurrenceSpec, ModelPlan, MoeFfnSpec, NormSpec, PositionSpec,
                   ScaledRopeSpec, ScheduleEntry, XieluFfnSpec)
from .registry import config_from_dict, config_from_json, register_architecture, supported_architectures
from .qwen2_moe import Qwen2MoeConfig
from .zusepel import ZusepelConfig
from .vumedra import VumedraConfig
from .migosun import MigosunConfig
from .sebevik import SebevikConfig

__all__ = ["AttentionSpec", "BlockSpec", "DecayBonusRecurrenceSpec", "DenseFfnSpec", "DepthMixBlockSpec",
           "LatentAttentionSpec", "LowerBoundRecurrenceSpec", "ModelPlan", "MoeFfnSpec", "NormSpec", "PositionSpec",
           "ScaledRopeSpec", "ScheduleEntry", "XieluFfnSpec", "ZusepelConfig", "VumedraConfig", "MigosunConfig", "SebevikConfig", "config_from_dict", "config_from_json", "register_architecture",
           "supported_architectures", "Qwen2MoeConfig"]
