"""b200moe: a Blackwell-native (sm_100a) distributed MoE training framework."""
__version__ = "0.1.0"
