"""pom_b200 — B200-native Polynomial Mixer layer (drop-in for ``pom.PoM`` / ``pom.PoMRoPE``)."""
from .functional import BlockCausal, SeqShard, polynomial_aggregation_, polynomial_selection_, pom
from .pom import PoM
from .pom_rope import PoMRoPE

__all__ = ["PoM", "PoMRoPE", "pom", "polynomial_aggregation_", "polynomial_selection_", "SeqShard", "BlockCausal"]
