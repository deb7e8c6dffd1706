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
