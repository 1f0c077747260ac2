"""primus_b200: a Blackwell-native (sm_100a) LLM pre-training framework."""
__version__ = "0.1.0"
