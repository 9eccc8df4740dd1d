from .base import (ArchEntry, ConfigError, arch_name_of, archs, find_arch, load_config,  # noqa: F401
                   read_config_json, register_arch)
from .qwen2_moe import Qwen2MoeConfig  # noqa: F401
