from .errors import (InvalidConfig, InvalidModelDir, MissingFile, ModelLoadError, UnsupportedDType, WeightError)
from .generation import DEFAULT_MAX_NEW_TOKENS, GenerationConfig, load_generation_config
from .metadata import (ModelMetadata, canonical_dtype, metadata_from_json, read_config_json, validate_run_dtype)
from .qwen3 import Qwen3Config
from .registry import (Architecture, architecture_for, register_architecture, registered_architectures,
                       spec_from_config_json, unregister_architecture)
from .fasesun import FasesunConfig
from .bisudra import BisudraConfig
from .pegurax import PeguraxConfig
from .nugolorn import NugolornConfig
from .specs import (AttentionSpec, BlockSpec, ChannelDecayMemorySpec, DeltaRuleSpec, DenseFeedForwardSpec, DifferentialAttentionSpec, MaskedAttentionSpec, SandwichBlockSpec,
                    ScaledRotationSpec, SelectiveScanSpec, SideBySideSpec, LatentAttentionSpec, LinearRecurrenceSpec, ModelSpec, NormSpec, PairRotationSpec,
                    PositionSpec, RoutedExpertsSpec, ScheduleEntry, SublayerNormBlockSpec, SwiGLUSpec, TokenSideSpec)
