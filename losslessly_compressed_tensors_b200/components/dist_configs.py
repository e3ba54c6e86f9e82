"""Default codebooks of the components (values of the reference's
``LCT/components/dist_configs.py:3-35``)."""
from ..comp_format import Distribution, DistType, NoiseLevel

weight_dist = Distribution(DistType.LAPLACE, noise_level=NoiseLevel.CLEAN)

# Momentum after the first step, and on the first step (many exact zeros).
momentum_dist = Distribution(DistType.EMPIRICAL, noise_level=NoiseLevel.CLEAN, zero_prob=0.02)
momentum_first_dist = Distribution(DistType.EMPIRICAL, noise_level=NoiseLevel.CLEAN, zero_prob=0.5)

act_dist = Distribution(DistType.LAPLACE, noise_level=NoiseLevel.CLEAN)
act_relu_dist = Distribution(DistType.LAPLACE, noise_level=NoiseLevel.CLEAN, zero_prob=0.5)
