from .model_config import (  # noqa: F401
    AttentionSpec,
    ConfigError,
    GatedMLPSpec,
    LayerRun,
    LayerSpec,
    LMHeadSpec,
    ModelConfig,
    PartSpec,
    RMSNormSpec,
    RotarySpec,
    TokenEmbeddingSpec,
    normalise_dtype,
    read_config_json,
)
from .registry import (  # noqa: F401
    ARCHITECTURES,
    Architecture,
    TensorNames,
    architecture_of,
    load_config,
    parse_config,
    register_architecture,
)
