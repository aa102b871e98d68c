"""nanoplm_b200: Blackwell-native protein language model pretraining and distillation."""
__version__ = "0.1.0"
