"""sirius_b200: B200-native colocated training step behind the Sirius torch_col surface."""
__all__ = ["ops", "_lib"]
