"""dawn_srw_b200: a Blackwell-native (B200, sm_100a) training and inference
framework for DAWN-SRW language models."""
__version__ = "0.1.0"

from .config import Config, load_config, preset  # noqa: F401
