"""Default codebooks of the components: the families and zero probabilities of the reference's
``LCT/components/dist_configs.py:3-35`` (all in the CLEAN layout)."""
from ..comp_format import Distribution, DistType, NoiseLevel


def _clean(family: DistType, zero_prob: float = 0.0) -> Distribution:
    return Distribution(family, noise_level=NoiseLevel.CLEAN, zero_prob=zero_prob)


weight_dist = _clean(DistType.LAPLACE)
act_dist = _clean(DistType.LAPLACE)
act_relu_dist = _clean(DistType.LAPLACE, 0.5)          # about half exact zeros after a ReLU
momentum_dist = _clean(DistType.EMPIRICAL, 0.02)       # optimizer state after the first step
momentum_first_dist = _clean(DistType.EMPIRICAL, 0.5)  # ... and on the first step (many zeros)
