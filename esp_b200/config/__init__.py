from .plan import (AttentionSpec, BlockSpec, DecayBonusRecurrenceSpec, DenseFfnSpec, DepthMixBlockSpec,
                   LatentAttentionSpec, LowerBoundRecurrenceSpec, ModelPlan, MoeFfnSpec, NormSpec, PositionSpec,
                   ScaledRopeSpec, ScheduleEntry, XieluFfnSpec)
from .registry import config_from_dict, config_from_json, register_architecture, supported_architectures
from .qwen2_moe import Qwen2MoeConfig
from .zusepel import ZusepelConfig

__all__ = ["AttentionSpec", "BlockSpec", "DecayBonusRecurrenceSpec", "DenseFfnSpec", "DepthMixBlockSpec",
           "LatentAttentionSpec", "LowerBoundRecurrenceSpec", "ModelPlan", "MoeFfnSpec", "NormSpec", "PositionSpec",
           "ScaledRopeSpec", "ScheduleEntry", "XieluFfnSpec", "ZusepelConfig", "config_from_dict", "config_from_json", "register_architecture",
           "supported_architectures", "Qwen2MoeConfig"]
