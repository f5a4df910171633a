"""Model families: weight containers, tensor-parallel sharding and the fp32 CPU oracle."""
from .llama import (FullWeights, RankWeights, LayerWeights, ReferenceLlama, random_full_weights,
                    shard_weights, random_rank_weights)
