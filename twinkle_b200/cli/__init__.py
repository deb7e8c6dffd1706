from .cli import CLI, Args, ArgGroup, GROUPS
