"""HTTP server: typed config, launcher, Gateway / Model / Sampler / Processor applications."""
from .config import ServerConfig
from .launcher import ServerLauncher, launch_server
from .state import ServerState
