from b200moe.utils.checkpoint import (_load_legacy_optimizer, _write_checkpoint, load_checkpoint,  # noqa: F401
                                      load_checkpoint_async_dist, move_model_state, move_optimizer_state,
                                      save_checkpoint, save_checkpoint_async_dist)
from b200moe.utils.data import get_batch, load_dataset  # noqa: F401


def compile_model(model):
    """The reference compiles three layer types with Inductor here
    (implementation/train_utils.py:34-43).  This framework's layers already run
    hand-written kernels, so there is nothing to compile; the model is returned
    unchanged."""
    return model
