from b200moe.config import (load_config, main, parallel_rank_groups, parallel_sizes,  # noqa: F401
                            validate_config, validate_router_aux_loss_coef)

if __name__ == "__main__":
    raise SystemExit(main())
