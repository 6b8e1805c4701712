"""aeris_gb_b200: a Blackwell-native (sm_100a) training and inference framework for the AERIS pixel-level Swin
diffusion weather model (TrigFlow), with window / sequence / pipeline / data parallelism on one NVSwitch box."""
__version__ = "0.1.0"
