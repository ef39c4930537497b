"""pom_b200 — B200-native Polynomial Mixer layer (drop-in for ``pom.PoM`` / ``pom.PoMRoPE``)."""
from .pom import PoM
from .pom_rope import PoMRoPE
# after the sub-modules, so that ``pom_b200.pom`` names the function as ``pom.pom`` does in the reference
# (pom/__init__.py: ``from .pom import PoM, pom``); the module stays importable as ``pom_b200.pom``
from .functional import BlockCausal, SeqShard, polynomial_aggregation_, polynomial_selection_, pom

__all__ = ["PoM", "PoMRoPE", "pom", "polynomial_aggregation_", "polynomial_selection_", "SeqShard", "BlockCausal"]
