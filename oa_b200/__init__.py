"""oa_b200: a Blackwell-native framework with the public surface of realminc/oa."""
__version__ = "0.1.0"
