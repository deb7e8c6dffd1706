from .device_mesh import DeviceGroup, DeviceMesh, is_last_rank, is_master
from .framework import Torch
from .import_utils import exists, requires
from .loader import Plugin, any_callable, check_unsafe, construct_class, trust_remote_code
from .logger import get_logger
from .misc import (align_logps_to_mask, call_with_supported_kwargs, copy_files_by_pattern, deep_getattr, find_all_linears, get_llm_model,
                   get_runtime_meta, has_signature_parameter, load_image, load_mm_file)
from .network import find_free_port, find_node_ip
from .platform import GPU, Platform
from .seed import stable_seed
from . import framework as framework_util
from . import torch_utils as torch_util
from .dequantizer import Dequantizer, dequant_fp8_block, dequant_mxfp4
from .parallel import file_lock as processing_lock
from .safetensors_io import SafetensorLazyLoader, StreamingSafetensorSaver
from .torch_utils import (clone_state_dict_to_cpu, pad_and_stack_tensors, pad_sequence_to_length, selective_log_softmax, to_device)
