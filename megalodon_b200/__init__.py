"""megalodon_b200: a Blackwell-native (sm_100a) Megalodon training and
inference framework."""
__version__ = "0.1.0"
