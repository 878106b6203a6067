"""Per-layer, per-epoch phase timers with the reference's names (time_recorder.py:5-211).

The reference brackets each phase with time.perf_counter() on the CPU.  GPU phases are
asynchronous, so a phase is bracketed with a pair of CUDA events instead
(`TimeRecorder.ctx.start()` / `record_*_time(token)`); the pairs are resolved to seconds when an
epoch closes, without stalling the stream in between.  Plain float durations are accepted too.
Recording is off (`enabled = False`) unless asked for: event bookkeeping is not free.
"""
import numpy as np
import torch
import torch.distributed as dist

_PHASES = ("barrier", "quantization", "communication", "dequantization", "prepare_comm", "pre_aggregate",
           "local_aggregate", "remote_aggregate", "total_covolution")


class TimeRecorder(object):
    ctx = None

    def __init__(self, num_layer, num_epoch, enabled: bool = False) -> None:
        for name in _PHASES:
            setattr(self, name + "_time", torch.zeros((num_layer * 2, num_epoch)))
        self.total_training_time = torch.zeros(num_epoch)
        self.cur_epoch = 0
        self.cur_layer = 0
        self._is_training = True
        self.enabled = enabled
        self._pending = []  # (tensor, layer, epoch, start_event, end_event)
        TimeRecorder.ctx = self

    # ---- event tokens -----------------------------------------------------------------------
    def start(self):
        """Open a phase on the current stream; returns a token for record_*_time, or None when
        recording is off or no GPU is in use."""
        if not (self.enabled and self._is_training and torch.cuda.is_available()):
            return None
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        return ev

    def _add(self, table: torch.Tensor, t) -> None:
        if not self._is_training or t is None:
            return
        if isinstance(t, torch.cuda.Event):
            end = torch.cuda.Event(enable_timing=True)
            end.record()
            self._pending.append((table, self.cur_layer, self.cur_epoch, t, end))
        elif table.dim() == 2:
            table[self.cur_layer, self.cur_epoch] += float(t)
        else:
            table[self.cur_epoch] += float(t)

    def _resolve(self) -> None:
        if not self._pending:
            return
        torch.cuda.synchronize()
        for table, layer, epoch, a, b in self._pending:
            sec = a.elapsed_time(b) / 1000.0
            if table.dim() == 2:
                table[layer, epoch] += sec
            else:
                table[epoch] += sec
        self._pending = []

    # ---- the reference's recording API ------------------------------------------------------
    def record_barrier_time(self, time) -> None:
        self._add(self.barrier_time, time)

    def record_quantization_time(self, time) -> None:
        self._add(self.quantization_time, time)

    def record_communication_time(self, time) -> None:
        self._add(self.communication_time, time)

    def record_dequantization_time(self, time) -> None:
        self._add(self.dequantization_time, time)

    def record_total_convolution_time(self, time) -> None:
        self._add(self.total_covolution_time, time)

    def record_prepare_comm_time(self, time) -> None:
        self._add(self.prepare_comm_time, time)

    def record_pre_aggregate_time(self, time) -> None:
        self._add(self.pre_aggregate_time, time)

    def record_local_aggregate_time(self, time) -> None:
        self._add(self.local_aggregate_time, time)

    def record_remote_aggregate_time(self, time) -> None:
        self._add(self.remote_aggregate_time, time)

    def record_total_training_time(self, time) -> None:
        self._add(self.total_training_time, time)

    def next_layer(self) -> None:
        if self._is_training:
            self.cur_layer += 1

    def next_epoch(self) -> None:
        if self._is_training:
            self._resolve()
            self.cur_epoch += 1
            self.cur_layer = 0

    def set_is_training(self, is_training: bool) -> None:
        self._is_training = is_training

    @staticmethod
    def print_time(rank, message, time):
        if rank == 0 and TimeRecorder.ctx is not None and getattr(TimeRecorder.ctx, "verbose", False):
            print("{}{}".format(message, time))

    # ---- totals in ms (time_recorder.py:72-103) ------------------------------------------------
    def _total(self, table) -> float:
        self._resolve()
        return torch.sum(table).item() * 1000.0

    def get_total_barrier_time(self) -> float:
        return self._total(self.barrier_time)

    def get_total_quantization_time(self) -> float:
        return self._total(self.quantization_time)

    def get_total_communication_time(self) -> float:
        return self._total(self.communication_time)

    def get_total_dequantization_time(self) -> float:
        return self._total(self.dequantization_time)

    def get_total_convolution_time(self) -> float:
        return self._total(self.total_covolution_time)

    def get_total_prepare_comm_time(self) -> float:
        return self._total(self.prepare_comm_time)

    def get_total_pre_aggregate_time(self) -> float:
        return self._total(self.pre_aggregate_time)

    def get_total_local_aggregate_time(self) -> float:
        return self._total(self.local_aggregate_time)

    def get_total_remote_aggregate_time(self) -> float:
        return self._total(self.remote_aggregate_time)

    def get_total_training_time(self) -> float:
        return self._total(self.total_training_time)

    def _reduced_totals(self):
        names = ("barrier", "quantization", "communication", "dequantization", "convolution", "prepare_comm",
                 "pre_aggregate", "local_aggregate", "remote_aggregate", "training")
        vals = torch.tensor([getattr(self, f"get_total_{n}_time")() for n in names], dtype=torch.float64)
        if dist.is_initialized() and dist.get_world_size() > 1:
            dev = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend() == "nccl" else vals.device
            v = vals.to(dev)
            dist.reduce(v, 0, op=dist.ReduceOp.SUM)
            vals = v.cpu() / dist.get_world_size()
        return dict(zip(names, vals.tolist()))

    def print_total_time(self) -> None:
        """Rank-0 summary of the mean (over ranks) total per phase, in ms (time_recorder.py:105-140)."""
        totals = self._reduced_totals()
        if not dist.is_initialized() or dist.get_rank() == 0:
            for name, v in totals.items():
                print("total_{}_time(ms): {}".format(name, v))

    def save_time_to_file(self, graph_name, world_size, out_dir: str = ".") -> None:
        """<phase>_time_<graph>_<world>.npy per phase, rank 0 only, mean over ranks
        (time_recorder.py:143-206)."""
        import os
        self._resolve()
        for name in _PHASES + ("total_training",):
            table = getattr(self, name + "_time").clone()
            if dist.is_initialized() and dist.get_world_size() > 1:
                dev = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend() == "nccl" else "cpu"
                t = table.to(dev)
                dist.reduce(t, 0, op=dist.ReduceOp.SUM)
                table = t.cpu() / dist.get_world_size()
            if not dist.is_initialized() or dist.get_rank() == 0:
                np.save(os.path.join(out_dir, "{}_time_{}_{}.npy".format(name, graph_name, world_size)),
                        table.numpy())
