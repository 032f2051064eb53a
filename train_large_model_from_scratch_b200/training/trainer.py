"""Training runtime: distributed init, data, model, optimizer, step loop,
evaluation, checkpointing, profiling and throughput/MFU reporting.

Public surface and overridable hooks follow the reference's `Trainer`
(`training/trainer.py:37-408`): `Trainer(config).train()`, `.eval()`,
`.save(step)`, `_init_distributed/_init_dataset/_init_model/_init_optimizer/
_init_profiler/_init_logging`, `_lr_scheduler`, `_one_training_micro_step`,
`_one_training_step`, `_resume_from_checkpoint`. Console line, `log.txt`
grammar (`"{step} train {loss:.6f}"`, `"{step} val {loss:.4f}"`), log-directory
name and checkpoint files are the same.

What is different underneath: there is no DDP wrapper and no autocast. The
model's parameters and gradients live in flat buffers; the optimizer step is
reduce-scatter -> global-norm clip -> fused AdamW -> all-gather over those
buffers (one pass for DP averaging, SP summation and ZeRO-1), and step time is
also measured on the device with CUDA events.
"""
from __future__ import annotations

import math
import os
import socket
import time
from collections import OrderedDict
from contextlib import contextmanager, nullcontext
from itertools import islice

import torch
import torch.distributed as dist

from ..models import GPT
from ..models.gpt import EXPERT_LOCAL_PARAM_SUFFIXES
from ..parallel import parallel_state
from ..parallel.zero1.distributed_optimizer import DistributedOptimizer, FusedAdamW
from ..utils import compute_mfu, get_model_params, get_training_info, set_seed
from ..utils.profile import get_measured_peak_flops
from ..utils.training import lr_schedule
from . import checkpoint as ckpt
from .config import Config
from .data import MockDataset, build_loader

try:
    from tqdm.auto import tqdm
except Exception:                                           # pragma: no cover
    tqdm = None


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


class Trainer:
    def __init__(self, config: Config):
        self.config = config
        self._init_distributed(config)
        t = config.train
        micro_tokens = t.batch_size * t.seq_len * self.dp_world_size
        assert t.total_batch_size % micro_tokens == 0, (
            f"make sure total_batch_size {t.total_batch_size} is divisible by batch_size {t.batch_size} * "
            f"seq_len {t.seq_len} * dp_world_size {self.dp_world_size}")
        if self.master_process:
            print(f"Training config: {config.as_dict()}")
        self._init_dataset(config)
        self.training_info = get_training_info(
            len(self.train_dataset), t.seq_len, t.total_batch_size, t.batch_size, self.dp_world_size,
            t.max_steps, t.max_epochs)
        if config.optim.warmup_steps >= self.training_info["max_steps"]:
            raise ValueError(f"warmup_steps must be < max_steps. Got warmup_steps={config.optim.warmup_steps}, "
                             f"max_steps={self.training_info['max_steps']}.")
        if self.master_process:
            print(f"The training process will train {self.training_info['epochs']} epochs, "
                  f"{self.training_info['max_steps']} steps.")
            print(f"=> calculated gradient accumulation steps: {self.training_info['grad_accum_steps']}")
            print(f"=> calculated tokens per step: {self.training_info['total_tokens_per_step']}")
        self._init_model(config)
        self._init_optimizer(config)
        self._init_logging(config)
        self.start_step = 0
        self.results = {}
        self.one_step_results = {}
        self.train_loader_iter = None
        self.profiler = None
        self.profiler_record_fn = self._null_record
        self.step_ms_device = None
        # CUDA-graph execution of the step (see `_train_step_graphed`)
        self._graph = None
        self._graph_in = None
        self._graph_out = None
        self._graph_launches = 0
        self._graph_eager_steps = 0
        self._graph_disabled = False
        self._prefetched = None            # next step's batches, already on their way to the device
        self._copy_stream = None

    # ------------------------------------------------------------------ init hooks
    def _init_distributed(self, config: Config) -> None:
        self.rank = int(os.environ.get("RANK", 0))
        self.local_rank = int(os.environ.get("LOCAL_RANK", 0))
        self.world_size = int(os.environ.get("WORLD_SIZE", 1))
        self.use_cuda = torch.cuda.is_available()
        backend = config.parallel.backend
        if backend == "nccl" and not self.use_cuda:
            backend = "gloo"
        self.backend = backend
        self._owns_pg = False
        if not dist.is_initialized():
            if config.parallel.init_method == "env://":
                os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
                os.environ.setdefault("MASTER_PORT", str(_free_port()))
                os.environ.setdefault("RANK", "0")
                os.environ.setdefault("WORLD_SIZE", "1")
            kwargs = {}
            if self.use_cuda and backend == "nccl":
                kwargs["device_id"] = torch.device("cuda", self.local_rank)
            import datetime
            kwargs["timeout"] = datetime.timedelta(seconds=float(config.parallel.dist_timeout_s))
            dist.init_process_group(backend=backend, init_method=config.parallel.init_method, **kwargs)
            self._owns_pg = True
        if self.use_cuda:
            torch.cuda.set_device(self.local_rank)
            self.device = torch.device("cuda", self.local_rank)
        else:
            self.device = torch.device("cpu")
        set_seed(config.seed.seed + self.rank, deterministic=config.seed.deterministic)
        self.master_process = self.rank == 0
        if not parallel_state.is_initialized():
            parallel_state.initialize_model_parallel(config=config.parallel)
        ps = parallel_state
        self.dp_group, self.dp_rank, self.dp_world_size = ps.get_dp_group(), ps.get_dp_rank(), ps.get_dp_world_size()
        self.sp_group, self.sp_rank, self.sp_world_size = ps.get_sp_group(), ps.get_sp_rank(), ps.get_sp_world_size()
        self.dp_sp_group, self.dp_sp_rank, self.dp_sp_world_size = (
            ps.get_dp_sp_group(), ps.get_dp_sp_rank(), ps.get_dp_sp_world_size())
        self.heartbeat = None
        if self.world_size > 1 and config.parallel.heartbeat_timeout_s > 0:
            from ..utils.health import Heartbeat
            self.heartbeat = Heartbeat(self.rank, self.world_size, config.parallel.heartbeat_timeout_s)

    def _init_dataset(self, config: Config) -> None:
        d, t = config.data, config.train
        if d.use_mock_data:
            self.train_dataset = MockDataset(d.mock_data_num_samples, t.seq_len, vocab_size=config.model.vocab_size,
                                             base_seed=config.seed.seed)
            self.val_dataset = (MockDataset(d.mock_data_num_samples // 10, t.seq_len,
                                            vocab_size=config.model.vocab_size, base_seed=config.seed.seed,
                                            seed_offset=1_000_000_000) if t.do_val else None)
        else:
            raise NotImplementedError(
                "no built-in on-disk dataset: pass --use_mock_data or subclass Trainer and override "
                "_init_dataset (see pretrain_example.py)")
        self._build_loaders(config)

    def _build_loaders(self, config: Config) -> None:
        d, t = config.data, config.train
        self.train_sampler, self.train_loader = build_loader(
            self.train_dataset, t.batch_size, self.dp_world_size, self.dp_rank, True, d.num_workers, d.pin_memory)
        if getattr(self, "val_dataset", None) is not None:
            self.val_sampler, self.val_loader = build_loader(
                self.val_dataset, t.batch_size, self.dp_world_size, self.dp_rank, False, d.num_workers, d.pin_memory)
        else:
            self.val_dataset = self.val_loader = None

    def _compute_dtype(self, precision: str) -> torch.dtype:
        if precision == "fp16":
            raise NotImplementedError("FP16 precision is not supported yet")
        if precision == "fp32" or not self.use_cuda:
            return torch.float32
        if precision == "bf16":
            return torch.bfloat16
        raise ValueError(f"Unsupported precision: {precision}. Supported precisions are: bf16, fp32.")

    def _init_model(self, config: Config) -> None:
        self.model_config = config.model
        if self.master_process:
            print(f"Params config: {get_model_params(self.model_config)}")
        from ..parallel import symm
        dtype = self._compute_dtype(config.train.precision)
        self._symm = symm.use_symm() and dtype == torch.bfloat16 and config.parallel.use_distributed_optimizer
        self.model = GPT(self.model_config, device=self.device, compute_dtype=dtype,
                         shard_world=self.dp_sp_world_size, alloc=symm.symm_alloc if self._symm else None)
        self.raw_model = self.model

    def _init_optimizer(self, config: Config) -> None:
        o = config.optim
        zero1 = config.parallel.use_distributed_optimizer
        m = self.raw_model
        # dense parameters are replicated over the whole world (their gradients are
        # summed over SP and averaged over DP); expert parameters only over DP.
        buffers = [m.dense_buf] + ([m.expert_buf] if m.expert_buf is not None else [])
        groups = [self.dp_sp_group] + ([self.dp_group] if m.expert_buf is not None else [])
        cuts = bucket_groups = None
        if zero1 and self.world_size > 1:
            # buckets of the sharded step: cut at layer groups of ~TLM_ZERO1_BUCKET_MB of fp32 gradients
            cuts, bucket_groups = m.plan_buckets(int(float(os.environ.get("TLM_ZERO1_BUCKET_MB", "192")) * (1 << 20)))
        fused = FusedAdamW(buffers, lr=o.max_lr, betas=(o.adam_beta1, o.adam_beta2), eps=o.adam_eps,
                           weight_decay=o.weight_decay, groups=groups, grad_divisor=self.dp_world_size,
                           sharded=zero1, norm_group=self.dp_sp_group, cuts=cuts, bucket_groups=bucket_groups)
        if getattr(self, "_symm", False):
            from ..parallel.symm import PeerCollectives
            fused._comm = PeerCollectives.create(fused, wire_dtype=config.parallel.grad_wire_dtype)
            if fused._comm.state:
                m.comm_hooks = fused          # forward: gate GEMMs on "parameters ready"; backward: start bucket reductions
        if zero1:
            named = OrderedDict((n, p) for n, p in m.named_parameters())
            self.optimizer = DistributedOptimizer(optimizer=fused, process_group=self.dp_group, named_tensors=named)
            self.raw_optimizer = self.optimizer.optimizer
        else:
            self.optimizer = self.raw_optimizer = fused

    @staticmethod
    @contextmanager
    def _null_record(name: str):
        yield

    def _init_profiler(self, config: Config) -> None:
        t = config.train
        if t.use_profiler:
            assert t.steps_to_profile[0] >= 1, "steps_to_profile[0] should be >= 1"
            acts = [torch.profiler.ProfilerActivity.CPU]
            if self.use_cuda:
                acts.append(torch.profiler.ProfilerActivity.CUDA)

            def on_ready(prof):
                if self.master_process:
                    prof.export_chrome_trace(f"{self.log_dir}/rank{self.rank}_trace.json")
            self.profiler = torch.profiler.profile(
                schedule=torch.profiler.schedule(wait=t.steps_to_profile[0] - 1, warmup=1,
                                                 active=t.steps_to_profile[1] + 1 - t.steps_to_profile[0], repeat=1),
                on_trace_ready=on_ready, record_shapes=True, with_stack=True, with_flops=True, activities=acts)
            self.profiler_record_fn = torch.profiler.record_function
        else:
            self.profiler = None
            self.profiler_record_fn = self._null_record

    def _init_logging(self, config: Config) -> None:
        n_params = sum(p.numel() for p in self.raw_model.parameters())
        self.log_dir = os.path.join(
            config.logging.log_dir,
            f"{config.logging.exp_name}_modelsize_{n_params}_lr{config.optim.max_lr}_BS{config.train.batch_size}_"
            f"SL{config.train.seq_len}_DP{self.dp_world_size}_SEP{parallel_state.get_sep_world_size()}_")
        self.log_file = os.path.join(self.log_dir, "log.txt")
        if self.master_process:
            os.makedirs(self.log_dir, exist_ok=True)
            resuming = ckpt.find_latest_complete(config.ckpt.resume_path or self.log_dir, self.rank) is not None
            if not resuming:
                open(self.log_file, "w").close()
        if self.world_size > 1:
            dist.barrier()

    # ------------------------------------------------------------------ schedule / precision
    def _lr_scheduler(self, it: int, max_steps: int, warmup_steps: int, max_lr: float, min_lr: float) -> float:
        return lr_schedule(it, max_steps, warmup_steps, max_lr, min_lr)

    def _autocast_context(self, precision: str):
        """Kept for API parity. Mixed precision is built into the ops (bf16
        GEMM inputs, fp32 residual/norm/loss), so no autocast is needed."""
        if precision == "fp16":
            raise NotImplementedError("FP16 precision is not supported yet")
        if precision not in ("bf16", "fp32"):
            raise ValueError(f"Unsupported precision: {precision}. Supported precisions are: bf16, fp32.")
        return nullcontext()

    # ------------------------------------------------------------------ steps
    def _sp_slice(self, x: torch.Tensor) -> torch.Tensor:
        T = x.shape[1]
        assert T % self.sp_world_size == 0, "sequence length must be divisible by sp_world_size"
        c = T // self.sp_world_size
        return x[:, self.sp_rank * c:(self.sp_rank + 1) * c]

    def _to_device(self, x: torch.Tensor) -> torch.Tensor:
        x = self._sp_slice(x)
        if x.device == self.device:
            return x.contiguous()
        if not self.use_cuda:
            return x.contiguous()
        if x.is_pinned() and self.sp_world_size == 1:
            return x.to(self.device, non_blocking=True)
        x = x.contiguous()
        if self.config.data.pin_memory:
            x = x.pin_memory()
        return x.to(self.device, non_blocking=True)

    def _batch_to_device(self, data_batch: dict):
        """(input_ids, labels) of this rank's sequence slice on the training device. Batches that `_prefetch`
        already sliced and copied are passed through."""
        if data_batch.get("_staged", False):
            return data_batch["input_ids"], data_batch["labels"]
        return self._to_device(data_batch["input_ids"]), self._to_device(data_batch["labels"])

    def _one_training_micro_step(self, config: Config, micro_step: int, data_batch: dict):
        x, y = self._batch_to_device(data_batch)
        ga = self.training_info["grad_accum_steps"]
        with self.profiler_record_fn("forward"):
            _, loss, logging_loss = self.model(x, y, loss_scale=1.0 / ga)
        with self.profiler_record_fn("backward"):
            loss.backward()
        return logging_loss.detach()

    def _next_batch(self) -> dict:
        if self.train_loader_iter is None:
            self.train_loader_iter = enumerate(self.train_loader)
        try:
            _, batch = next(self.train_loader_iter)
        except StopIteration:
            self._epoch = getattr(self, "_epoch", 0) + 1
            self.train_sampler.set_epoch(self._epoch)
            self.train_loader_iter = enumerate(self.train_loader)
            _, batch = next(self.train_loader_iter)
        return batch

    # ------------------------------------------------------------------ input prefetch
    def _prefetch(self) -> None:
        """Fetch the NEXT step's micro-batches from the loader, slice this rank's part of the sequence, stage
        it in pinned memory and start its host->device copy on a side stream. Called right after a step's
        device work has been queued, so that the loader's host work and the copy run under that step's
        kernels (the reference copies each batch synchronously in front of its forward pass,
        `training/trainer.py:227-228`)."""
        if not self.use_cuda or os.environ.get("TLM_PREFETCH", "1") == "0":
            return
        ga = self.training_info["grad_accum_steps"]
        host = [self._next_batch() for _ in range(ga)]
        if self._copy_stream is None:
            self._copy_stream = torch.cuda.Stream(device=self.device)
        staged = []
        with torch.cuda.stream(self._copy_stream):
            for b in host:
                x, y = self._sp_slice(b["input_ids"]).contiguous(), self._sp_slice(b["labels"]).contiguous()
                if not x.is_pinned():
                    x, y = x.pin_memory(), y.pin_memory()
                staged.append({"input_ids": x.to(self.device, non_blocking=True),
                               "labels": y.to(self.device, non_blocking=True), "_staged": True, "_pinned": (x, y)})
            ready = torch.cuda.Event()
            ready.record(self._copy_stream)
        self._prefetched = (staged, ready)

    def _take_prefetched(self):
        """The batches `_prefetch` staged (the current stream is made to wait for their copies), or None."""
        if self._prefetched is None:
            return None
        staged, ready = self._prefetched
        self._prefetched = None
        torch.cuda.current_stream().wait_event(ready)
        for b in staged:                      # the copies ran on the side stream: tie the tensors to this one as well
            b["input_ids"].record_stream(torch.cuda.current_stream())
            b["labels"].record_stream(torch.cuda.current_stream())
        return staged

    def _one_training_step(self, config: Config, step: int, batches: list | None = None) -> None:
        self.model.train()
        self.optimizer.zero_grad()
        loss_accum = None
        if batches is None:
            batches = self._take_prefetched()
        for micro_step in range(self.training_info["grad_accum_steps"]):
            batch = batches[micro_step] if batches is not None else self._next_batch()
            self.raw_optimizer.last_micro_step = micro_step == self.training_info["grad_accum_steps"] - 1
            l = self._one_training_micro_step(config, micro_step, batch)
            loss_accum = l if loss_accum is None else loss_accum + l
        lr = self._lr_scheduler(step, self.training_info["max_steps"], config.optim.warmup_steps,
                                config.optim.max_lr, config.optim.min_lr)
        for group in self.optimizer.param_groups:
            group["lr"] = lr
        norm = self.optimizer.step(grad_clip_value=config.train.grad_clip_value)
        if self.dp_world_size > 1:
            dist.all_reduce(loss_accum, op=dist.ReduceOp.SUM, group=self.dp_group)
            loss_accum = loss_accum / self.dp_world_size
        self.one_step_results["lr"] = lr
        self.one_step_results["loss"] = loss_accum
        self.one_step_results["grad_norm"] = norm

    # ------------------------------------------------------------------ the step as a CUDA graph
    def _graph_eligible(self) -> bool:
        """The whole step (zero-grad, every micro-step's forward and backward, reduce-scatter, clipped AdamW,
        all-gather, loss reduction) is recorded once and replayed when nothing in it needs the host: CUDA, bf16,
        and either one rank or the peer-memory collectives (library collectives stay un-recorded). The reference's
        `--use_compile` asks for its tracing compiler (`training/trainer.py:130-131`); here the flag is accepted
        and this launch-free replay is what speeds the step up, whether or not the flag is given.
        `TLM_CUDA_GRAPH=0` turns it off."""
        if self._graph_disabled or not self.use_cuda or os.environ.get("TLM_CUDA_GRAPH", "1") == "0":
            return False
        if self._compute_dtype(self.config.train.precision) != torch.bfloat16:
            return False
        if self.world_size > 1 and not getattr(self, "_symm", False):
            return False
        return not self.config.train.use_profiler

    def _device_step(self):
        """Everything of one optimizer step that runs on the device, reading the static input buffers."""
        cfg = self.config
        ga = self.training_info["grad_accum_steps"]
        self.model.train()
        self.optimizer.zero_grad()
        loss_accum = None
        for ms in range(ga):
            b = self._graph_in[ms]
            self.raw_optimizer.last_micro_step = ms == ga - 1
            _, loss, logging_loss = self.model(b["input_ids"], b["labels"], loss_scale=1.0 / ga)
            loss.backward()
            l = logging_loss.detach()
            loss_accum = l if loss_accum is None else loss_accum + l
        norm = self.optimizer.step_device(grad_clip_value=cfg.train.grad_clip_value)
        if self.dp_world_size > 1:
            from ..parallel.symm import scalar_all_reduce
            loss_accum = scalar_all_reduce(loss_accum, self.dp_group, 1.0 / self.dp_world_size)
        return loss_accum, norm

    def _train_step_graphed(self, step: int, batches: list | None) -> bool:
        """Runs the step from static buffers: eagerly for the first two calls (lazy set-up: symmetric buffers,
        kernel attributes, tables), then records it and replays the recording. Returns False if this step has to
        take the ordinary path (shape change, recording failed)."""
        from ..ops import native
        cfg = self.config
        ga = self.training_info["grad_accum_steps"]
        if batches is None:
            batches = self._take_prefetched()
        host = batches if batches is not None else [self._next_batch() for _ in range(ga)]
        xs = [((b["input_ids"], b["labels"]) if b.get("_staged", False)
               else (self._sp_slice(b["input_ids"]), self._sp_slice(b["labels"]))) for b in host]
        if self._graph_in is None:
            self._graph_in = [{"input_ids": torch.empty(x.shape, dtype=torch.int64, device=self.device),
                               "labels": torch.empty(y.shape, dtype=torch.int64, device=self.device)} for x, y in xs]
        if len(xs) != len(self._graph_in) or any(x.shape != g["input_ids"].shape for (x, _), g in zip(xs, self._graph_in)):
            self._pending_batches = host
            return False
        for (x, y), g in zip(xs, self._graph_in):
            if cfg.data.pin_memory and not x.is_cuda and not x.is_pinned():
                x, y = x.contiguous().pin_memory(), y.contiguous().pin_memory()
            g["input_ids"].copy_(x, non_blocking=True)
            g["labels"].copy_(y, non_blocking=True)
        lr = self._lr_scheduler(step, self.training_info["max_steps"], cfg.optim.warmup_steps, cfg.optim.max_lr,
                                cfg.optim.min_lr)
        for group in self.optimizer.param_groups:
            group["lr"] = lr
        self.optimizer.prepare_step()
        if self._graph is None and self._graph_eager_steps < 2:
            self._graph_eager_steps += 1
            loss, norm = self._device_step()
        else:
            if self._graph is None:
                torch.cuda.synchronize()
                graph = torch.cuda.CUDAGraph()
                before = native.launch_count()
                err = None
                try:
                    with torch.cuda.graph(graph, capture_error_mode="thread_local"):
                        self._graph_out = self._device_step()
                except Exception as e:                                   # keep training on the ordinary path
                    import traceback
                    err = (f"{type(e).__name__}: {str(e).splitlines()[0] if str(e) else ''}\n"
                           + "".join(traceback.format_exc().splitlines(keepends=True)[-14:]))
                # Every rank must take the same decision: the kernels of a replayed step and of an ordinary step
                # count the same flag epochs, but a rank that replays while another one re-runs its set-up
                # collectives would wait for exchanges the other never starts.
                if not self._all_ranks_ok(err is None):
                    self._graph_disabled = True
                    self._graph_out = None
                    if err is not None:
                        print(f"[warn] rank {self.rank}: recording the step as a CUDA graph failed ({err}); "
                              f"all ranks continue without it")
                    torch.cuda.synchronize()
                    loss, norm = self._device_step()
                    self.one_step_results.update(lr=lr, loss=loss, grad_norm=norm)
                    return True
                self._graph_launches = native.launch_count() - before
                self._graph = graph
            self._graph.replay()
            native.add_launch_count(self._graph_launches)
            # the recording writes its results into the same two tensors every time: hand out copies
            loss, norm = (t.clone() for t in self._graph_out)
        self.one_step_results.update(lr=lr, loss=loss, grad_norm=norm)
        return True

    def _all_ranks_ok(self, ok: bool) -> bool:
        """Logical AND of `ok` over all ranks (a host-side collective; call outside of stream capture)."""
        if self.world_size == 1:
            return ok
        t = torch.tensor([1 if ok else 0], dtype=torch.int32, device=self.device)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        return bool(t.item())

    def _read_device_status(self) -> int:
        """Status word of the kernels' bounded waits (0 = no wait ran out) since the last call. It lives in
        mapped host memory, so reading it costs nothing; the caller has synchronised."""
        if not self.use_cuda:
            return 0
        from ..ops import native
        return native.take_device_status() if native.available() else 0

    def _check_device_status(self) -> None:
        """After a step's synchronize: a kernel that gave up on a flag or barrier wait skipped its exchange
        (stale gradient shard, norm 0), so the step must not be committed. Raises `DeviceTimeout` and tells
        the peers through the heartbeat store."""
        st = self._read_device_status()
        if st:
            from ..utils.health import DeviceTimeout
            err = DeviceTimeout(st)
            if self.heartbeat is not None:
                self.heartbeat.announce_failure(str(err))
            raise err

    def train_step(self, step: int, batches: list | None = None) -> dict:
        """One optimizer step (all micro-steps). Public entry for callers that
        drive the loop themselves; returns `{lr, loss, grad_norm}` with `loss`
        and `grad_norm` as 0-d tensors on the training device. `batches`
        (optional) is a list of `grad_accum_steps` dicts with full-sequence
        `input_ids` / `labels`; by default the trainer's own loader is used."""
        self.one_step_results = {}
        hb = self.heartbeat
        if hb is not None:
            # learn about a dead or stalled peer on the host, before any kernel or collective of this step
            hb.enter_step(step)
        try:
            done = self._graph_eligible() and self._train_step_graphed(step, batches)
            if not done:
                pend = getattr(self, "_pending_batches", None)
                self._pending_batches = None
                self._one_training_step(self.config, step, batches if pend is None else pend)
            if batches is None and step + 1 < self.training_info["max_steps"]:
                self._prefetch()                   # host work + H2D copy of the next step, under this step's kernels
        except BaseException as e:
            if hb is not None:
                hb.announce_failure(f"{type(e).__name__}: {e}")
            raise
        if hb is not None:
            if self.use_cuda:
                torch.cuda.synchronize()
                self._check_device_status()
            hb.beat(step)
        return self.one_step_results

    # ------------------------------------------------------------------ resume / save
    def _steps_per_epoch(self) -> int:
        return max(1, len(self.train_loader) // self.training_info["grad_accum_steps"])

    def _resume_from_checkpoint(self, steps_per_epoch: int | None = None) -> None:
        ckpt_dir = self.config.ckpt.resume_path or self.log_dir
        prefix = ckpt.find_latest_complete(ckpt_dir, self.rank)
        if self.world_size > 1:                         # all ranks must agree
            objs = [prefix]
            dist.broadcast_object_list(objs, src=0)
            prefix = objs[0]
        if prefix is None:
            self.start_step = 0
            return
        meta = torch.load(f"{prefix}_meta.pt", map_location="cpu", weights_only=False)
        state = torch.load(f"{prefix}_model.pt", map_location="cpu", weights_only=True)
        ckpt.load_model_state_dict(self.raw_model, self.optimizer, state)
        key = f"optimizer/rank{self.rank}"
        placeholder = {key: ckpt.optimizer_state_dict(self.raw_model, self.optimizer)}
        ckpt.dcp_load(placeholder, f"{prefix}_opt")
        ckpt.load_optimizer_state_dict(self.raw_model, self.optimizer, placeholder[key])
        sampler_state = meta.get("sampler_state", {})
        epoch, iter_idx = sampler_state.get("epoch", 0), sampler_state.get("iter_idx", 0)
        self._epoch = epoch
        self.train_sampler.set_epoch(epoch)
        self.train_loader_iter = enumerate(islice(self.train_loader, iter_idx, None), start=iter_idx)
        step = meta.get("step")
        self.start_step = step + 1 if step is not None else 0
        if self.master_process:
            print(f"=> Resumed from {ckpt_dir} | next_step={self.start_step}, sampler_epoch={epoch}, "
                  f"dataloader_iter_idx={iter_idx}")
        rng_path = f"{prefix}_rng_rank{self.rank}.pt"
        if os.path.exists(rng_path):
            ckpt.set_rng_state(torch.load(rng_path, map_location="cpu", weights_only=False), self.local_rank)
        if self.world_size > 1:
            dist.barrier()
        if self.use_cuda:
            torch.cuda.synchronize()

    def save(self, step: int | None = None) -> None:
        step = 0 if step is None else step
        os.makedirs(self.log_dir, exist_ok=True)
        prefix = os.path.join(self.log_dir, f"{step:05d}")
        spe = self._steps_per_epoch()
        ga = self.training_info["grad_accum_steps"]
        nxt = step + 1
        sampler_state = {"epoch": nxt // spe, "iter_idx": (nxt % spe) * ga}
        model_state = ckpt.full_model_state_dict(self.raw_model, self.optimizer)        # collective
        opt_state = ckpt.optimizer_state_dict(self.raw_model, self.optimizer)           # collective
        ckpt.dcp_save({f"optimizer/rank{self.rank}": opt_state}, f"{prefix}_opt")
        rng = ckpt.rng_state(self.local_rank)
        ckpt._atomic_save(rng, f"{prefix}_rng_rank{self.rank}.pt")
        if self.world_size > 1:
            dist.barrier()
        if self.master_process:
            ckpt._atomic_save(model_state, f"{prefix}_model.pt")
            results = {k: (v.detach().cpu() if torch.is_tensor(v) else v) for k, v in self.one_step_results.items()}
            meta = {
                "trainer_config": self.config.as_dict(),
                "model_config": self.raw_model.config.as_dict(),
                "step": step,
                "this_step_results": results,
                "opt_part_assignment": getattr(self.optimizer, "part_assignment", None),
                "sampler_state": sampler_state,
                "rng_state": rng,
            }
            ckpt._atomic_save(meta, f"{prefix}_meta.pt")                               # commit marker, last
        if self.world_size > 1:
            dist.barrier()

    # ------------------------------------------------------------------ loops
    def train(self) -> None:
        cfg = self.config
        self.results = {}
        self.train_loader_iter = enumerate(self.train_loader)
        self._resume_from_checkpoint(self._steps_per_epoch())
        self._init_profiler(cfg)
        if self.profiler:
            self.profiler.start()
        max_steps = self.training_info["max_steps"]
        ga = self.training_info["grad_accum_steps"]
        steps = range(self.start_step, max_steps)
        bar = tqdm(steps, initial=self.start_step, total=max_steps, desc="Train",
                   disable=not self.master_process) if tqdm is not None else steps
        write = tqdm.write if tqdm is not None else print
        measured_peak = get_measured_peak_flops()
        for step in bar:
            t0 = time.time()
            last_step = step == max_steps - 1
            if self.use_cuda:
                ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                ev0.record()
            with self.profiler_record_fn("training_step"):
                self.train_step(step)
            if self.use_cuda:
                ev1.record()
                torch.cuda.synchronize()
                self.step_ms_device = ev0.elapsed_time(ev1)
            self._check_device_status()            # before logging, evaluation and save(): never commit a bad step
            if self.profiler:
                self.profiler.step()
            if not cfg.train.debug and cfg.train.do_val and (step % cfg.train.val_every_steps == 0 or last_step):
                self.eval()
                if self.master_process:
                    write(f"validation loss: {self.one_step_results['val_loss'].item():.4f}")
                    with open(self.log_file, "a") as f:
                        f.write(f"{step} val {self.one_step_results['val_loss'].item():.4f}\n")
            if cfg.ckpt.do_save and not cfg.train.debug and step > 0 and (
                    step % cfg.ckpt.save_every_steps == 0 or last_step):
                self.save(step)
            if self.heartbeat is not None:
                self.heartbeat.beat(step)          # evaluation and saving can outlast the heartbeat limit
            dt = time.time() - t0
            tokens = cfg.train.batch_size * cfg.train.seq_len * ga * self.dp_world_size
            mfu, _, _ = compute_mfu(self.raw_model, cfg.train.batch_size, cfg.train.seq_len, dt, ga, dtype="bf16") \
                if self.use_cuda else (0.0, 0.0, 0.0)
            if self.master_process:
                loss_v = float(self.one_step_results["loss"])
                extra = ""
                if self.use_cuda and measured_peak:
                    m2, _, _ = compute_mfu(self.raw_model, cfg.train.batch_size, cfg.train.seq_len, dt, ga,
                                           peak_flops=measured_peak)
                    extra = f" | MFU(measured peak): {m2 * 100:.2f}% | dt(device): {self.step_ms_device:.2f}ms"
                write(f"step {step:5d} | loss: {loss_v:.6f} | lr {self.one_step_results['lr']:.4e} | "
                      f"grad norm: {float(self.one_step_results['grad_norm']):.4f} | dt: {dt * 1000:.2f}ms | "
                      f"tok/sec: {tokens / dt:.2f} | MFU: {mfu * 100:.2f}%{extra}")
                with open(self.log_file, "a") as f:
                    f.write(f"{step} train {loss_v:.6f}\n")
            self.results[step] = dict(self.one_step_results)
        if self.profiler:
            self.profiler.stop()
        self.close()

    def close(self) -> None:
        if self._owns_pg and dist.is_initialized():
            parallel_state.destroy_model_parallel()
            dist.destroy_process_group()
            self._owns_pg = False

    @torch.no_grad()
    def eval(self) -> None:
        self.model.eval()
        n = len(self.val_loader)
        acc = None
        it = self.val_loader
        if tqdm is not None:
            it = tqdm(it, desc="Val", disable=not self.master_process)
        for batch in it:
            x, y = self._to_device(batch["input_ids"]), self._to_device(batch["labels"])
            _, _, logging_loss = self.model(x, y, loss_scale=1.0 / n)
            acc = logging_loss if acc is None else acc + logging_loss
        if self.use_cuda:
            torch.cuda.synchronize()
        if self.dp_world_size > 1:
            dist.all_reduce(acc, op=dist.ReduceOp.SUM, group=self.dp_group)
            acc = acc / self.dp_world_size
        self.one_step_results["val_loss"] = acc
