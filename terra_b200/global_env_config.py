"""Import-time environment flags (same names as the reference's core/global_env_config.py:5-164)."""
import os


def _flag(name, default="0"):
    return os.environ.get(name, default).strip().lower() in ("1", "true", "yes", "on")


ON_H200 = _flag("TERRA_ON_H200")                 # sequential model takes NCHW inputs when set
ENABLE_TORCH_PROF = _flag("ENABLE_TORCH_PROF")
DISABLE_TORCH_PROF = _flag("DISABLE_TORCH_PROF")
TORCH_PROF_WRITE_TRACE = _flag("TORCH_PROF_WRITE_TRACE")
TORCH_PROF_STEP_LIST = [int(v) for v in os.environ.get("TORCH_PROF_STEP_LIST", "1,1,3,1").split(",")]
DEBUG_GRAD_HOOK = _flag("DEBUG_GRAD_HOOK")
DEBUG_GRAD_HOOK_PRINT_LIMIT = int(os.environ.get("DEBUG_GRAD_HOOK_PRINT_LIMIT", "20"))
FSDP_WRAPPER_CFG = int(os.environ.get("FSDP_WRAPPER_CFG", "1"))
TERRA_USE_FAKE_INPUT = _flag("TERRA_USE_FAKE_INPUT")
USE_FAKE_INPUT = TERRA_USE_FAKE_INPUT            # the reference's name for the same switch
USE_FLASH_ATTENTION = "no use now"               # kept for code that imports it; attention has one implementation per device
TERRA_ALLOW_UNALIGNED_CROSS_NODE_WP = _flag("TERRA_ALLOW_UNALIGNED_CROSS_NODE_WP")

MEM_PROF = 0
use_Transformer = True
use_MLP = True
use_layernorm = True
use_shift_size_0 = False
emb_cfg = 4
EMB_1_input_split = EMB_1_output_split = EMB_2_input_split = EMB_2_output_split = "(m,1)"
EMB_1_SPLIT_PARAM = EMB_2_SPLIT_PARAM = True
