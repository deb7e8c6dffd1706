from .config import PRESETS, DecoderConfig, preset
from .decoder import DecoderModel, PackedBatch, build_model
from .layers import Linear, LoraBatch, RMSNorm, lora_batch
