"""Hand-written CUDA for sm_100a and its Python face (`kernels`)."""
from . import build, libraries  # noqa: F401
