"""astrai_b200: a Blackwell-native (sm_100a) transformer training and serving framework."""

__version__ = "0.1.0"
