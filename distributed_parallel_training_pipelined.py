"""torchrun entry point, same module name and ``--config-path`` flag as the
reference: ``torchrun … --module distributed_parallel_training_pipelined
--config-path configs/run_config.yaml``.  The worker lives in ``b200moe.trainer``."""
from b200moe.trainer import (_latest_checkpoint, _nvtx_range, _select_checkpoint,  # noqa: F401
                             _verify_pending_checkpoints, main, train)

if __name__ == "__main__":
    main()
