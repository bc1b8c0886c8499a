"""gin-config compatible configuration (see `t5x_b200.gin.config`)."""
from t5x_b200.gin.config import (  # noqa: F401
    REQUIRED, GinError, add_config_file_search_path, bind_parameter, clear_config, config_is_locked,
    config_scope, config_str, configurable, constant, external_configurable, finalize,
    get_configurable, markdown, operative_config_str, parse_config, parse_config_file,
    parse_config_files_and_bindings, parse_value, query_parameter, register, set_main_module)
