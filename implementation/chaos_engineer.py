from b200moe.utils.chaos import (CHAOS_FUNCTIONS, ChaosEnginnerTrigger, _cpu_burn, function_register,  # noqa: F401
                                 random_cpu_hog, random_delay, random_gpu_memory_leak, random_kill)
