"""brain_b200 — a B200-native (sm_100a) training and serving framework."""
__version__ = "0.1.0"
