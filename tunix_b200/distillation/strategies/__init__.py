from .base_strategy import BaseStrategy
from .logit import LogitStrategy
from .attention import AttentionTransferStrategy
from .feature_pooling import FeaturePoolingStrategy
from .feature_projection import FeatureProjectionStrategy
