"""Child process body for the multi-rank CPU tests: run the Trainer, dump losses."""
import json
import os
import sys

import torch

from train_large_model_from_scratch_b200.training import Trainer, build_config, parse_args


def main():
    torch.set_num_threads(2)
    args = parse_args(sys.argv[1:])
    cfg = build_config(args)
    t = Trainer(cfg)
    stop_after = int(os.environ.get("TLM_STOP_AFTER", "-1"))
    if stop_after >= 0:                      # emulate a job that ends early (checkpoint tests)
        t.training_info["max_steps_run"] = stop_after
    rank = t.rank
    t.train_loader_iter = enumerate(t.train_loader)
    t._resume_from_checkpoint()
    losses, norms = {}, {}
    last = t.training_info["max_steps"] if stop_after < 0 else stop_after
    exit_rank, exit_step = int(os.environ.get("TLM_EXIT_RANK", "-1")), int(os.environ.get("TLM_EXIT_BEFORE_STEP", "-1"))
    marker = os.environ.get("TLM_EXIT_ONCE_MARKER")
    for step in range(t.start_step, last):
        if rank == exit_rank and step == exit_step and not (marker and os.path.exists(marker)):
            # a host-made failure: this rank leaves between steps, with nothing in flight
            if marker:
                open(marker, "w").close()
            os._exit(17)
        r = t.train_step(step)
        losses[step] = float(r["loss"])
        norms[step] = float(r["grad_norm"])
        if cfg.ckpt.do_save and step > 0 and (step % cfg.ckpt.save_every_steps == 0):
            t.save(step)
    crash = os.environ.get("TLM_CRASH_IN_SAVE")
    if crash:
        import train_large_model_from_scratch_b200.training.checkpoint as ck
        orig = ck._atomic_save

        def failing(obj, path):
            if path.endswith("_meta.pt"):
                raise RuntimeError("injected failure before the commit marker")
            return orig(obj, path)
        ck._atomic_save = failing
        try:
            t.save(last - 1 + 100)
        except RuntimeError:
            pass
    wsum = float(t.raw_model.dense_buf.params.double().sum())
    guards = []
    if torch.cuda.is_available():
        from train_large_model_from_scratch_b200.ops import native
        from train_large_model_from_scratch_b200.parallel import symm
        torch.cuda.synchronize()
        guards = symm.check_guards()                     # empty unless TLM_SYMM_CANARY=1 found damage
        if native.available():
            native.raise_on_device_status()
        if t.world_size > 1:
            import torch.distributed as dist
            all_guards = [None] * t.world_size
            dist.all_gather_object(all_guards, guards)
            guards = [f"rank {r}: {g}" for r, gs in enumerate(all_guards) for g in gs]
    if rank == 0:
        with open(os.environ["TLM_TEST_OUT"], "w") as f:
            json.dump({"losses": losses, "norms": norms, "start_step": t.start_step, "wsum": wsum,
                       "log_dir": t.log_dir, "guards": guards}, f)
    t.close()


if __name__ == "__main__":
    main()
