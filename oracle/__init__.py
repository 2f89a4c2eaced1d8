"""CPU oracle of the training hot path: test infrastructure, never imported by the shipped package."""
from .oracle import ACT, COST, LMConfig, Oracle, build, pt_matrix, pt_positive_vector, pt_tensor3, pt_vector  # noqa: F401
