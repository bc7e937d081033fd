"""legion_b200: a Blackwell-native (B200, sm_100a) mixture-of-experts LLM inference engine."""
__version__ = "0.1.0"
