from .io import (load_checkpoint, save_checkpoint, read_global_step, checkpoint_dir, model_states_name,
                 optim_states_name, finalize_async_save)

__all__ = ["load_checkpoint", "save_checkpoint", "read_global_step", "checkpoint_dir", "model_states_name",
           "optim_states_name", "finalize_async_save"]
