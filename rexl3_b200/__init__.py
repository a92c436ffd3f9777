"""rexl3_b200: a Blackwell-native (sm_100a) EXL3 inference engine."""
__version__ = "0.1.0"
