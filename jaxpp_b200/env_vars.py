"""Flag objects under the names the reference exports them (src/jaxpp/env_vars.py:3-22)."""
from .utils.config import (conservative_loop_clustering as jaxpp_conservative_loop_clustering,
                           debug_force_mpmdify as jaxpp_debug_force_mpmdify,
                           debug_skip_propagation as jaxpp_debug_skip_propagation,
                           directional_communicators as jaxpp_directional_communicators,
                           disable_prevent_cse as jaxpp_disable_prevent_cse,
                           disable_schedule_task_fusion as jaxpp_disable_schedule_task_fusion,
                           dump_dir as jaxpp_dump_dir,
                           enable_licm as jaxpp_enable_licm,
                           enable_local_propagation as jaxpp_enable_local_propagation,
                           fast_infer_shardings as jaxpp_fast_infer_shardings,
                           share_donation as jaxpp_share_donation,
                           transfer_done_delay as jaxpp_transfer_done_delay)
