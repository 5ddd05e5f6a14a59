"""alpacca_b200: a small model library with generation of its own, for one
NVIDIA B200, built from what jtiro232/Alpacca's engine computes."""

__version__ = "0.1.0"
