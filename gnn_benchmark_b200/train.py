"""Full-batch training loop with the reference's structure and epoch log line
(self_benchmark/a64fx/train.py:19-109), on CUDA tensors.

    torchrun --nproc-per-node N -m gnn_benchmark_b200.train --config cfg.yaml --num_bits 2 --is_pre_delay true
"""
import argparse
import time

import torch
import torch.distributed as dist
import torch.nn.functional as F

from . import dense
from .communicator import Communicator
from .data_manager import load_data
from .model import create_model_and_optimizer, set_random_seed
from .quantizer import Quantizer_for_all_procs
from .time_recorder import TimeRecorder


def _world():
    return dist.get_world_size() if dist.is_initialized() else 1


def collect_acc(model, data):
    """train / val / test accuracy summed over ranks (train.py:19-40)."""
    TimeRecorder.ctx.set_is_training(False)
    model.eval()
    with torch.no_grad():
        out = model(data["graph"], data["nodes_features"])
    counts = []
    for mask in (data["nodes_train_masks"], data["nodes_valid_masks"], data["nodes_test_masks"]):
        correct = (out[mask].argmax(-1) == data["nodes_labels"][mask]).sum() if mask.size(0) != 0 else \
            torch.zeros((), dtype=torch.int64, device=out.device)
        counts += [correct.to(torch.int64), torch.tensor(mask.size(0), dtype=torch.int64, device=out.device)]
    counts = torch.stack(counts)
    if _world() > 1:
        dist.all_reduce(counts, op=dist.ReduceOp.SUM)
    c = counts.tolist()
    TimeRecorder.ctx.set_is_training(True)
    return tuple(c[i] / max(c[i + 1], 1) for i in (0, 2, 4))


def train(model, data, optimizer, num_epochs, num_bits, eval_every_epoch=True, log=print):
    """Returns (per-epoch loss list, per-epoch time list in s).  The timed region of an epoch is
    forward start -> optimiser step end, as in the reference (train.py:84-98), closed by a device
    synchronisation so that it covers the GPU work."""
    rank = dist.get_rank() if dist.is_initialized() else 0
    world_size = _world()
    losses, times = [], []
    if world_size > 1:
        dist.barrier()
    for epoch in range(num_epochs):
        model.train()
        torch.cuda.synchronize()
        forward_start = time.perf_counter()
        optimizer.zero_grad()
        out = model(data["graph"], data["nodes_features"])
        loss = F.nll_loss(out[data["nodes_train_masks"]], data["nodes_labels"][data["nodes_train_masks"]])
        loss.backward()
        optimizer.step()
        torch.cuda.synchronize()
        update_weight_end = time.perf_counter()
        dense.check_status()  # a tensor-core kernel that gave up on a bounded wait left its output partly written
        losses.append(float(loss.detach()))
        times.append(update_weight_end - forward_start)
        train_acc = val_acc = test_acc = float("nan")
        if eval_every_epoch:
            train_acc, val_acc, test_acc = collect_acc(model, data)
        if rank == 0 and log is not None:
            log(f"Rank: {rank}, World_size: {world_size}, Epoch: {epoch}, Loss: {losses[-1]}, Train: {train_acc:.4f}, "
                f"Val: {val_acc:.4f}, Test: {test_acc:.4f}, Time: {times[-1]:.6f}")
        TimeRecorder.ctx.record_total_training_time(times[-1])
        TimeRecorder.ctx.next_epoch()
    return losses, times


def main():
    import yaml

    parser = argparse.ArgumentParser()
    parser.add_argument("--config", type=str, default="config.yaml")
    parser.add_argument("--num_bits", type=int, default=32)
    parser.add_argument("--is_pre_delay", type=str, default="false")
    args = parser.parse_args()
    with open(args.config) as f:
        config = yaml.safe_load(f)
    config["num_bits"] = args.num_bits
    config["is_pre_delay"] = args.is_pre_delay == "true"

    Communicator(config["num_bits"], config.get("is_async", True))
    rank, world_size = Communicator.ctx.init_dist_group()
    Quantizer_for_all_procs(world_size, config["num_bits"])
    config["input_dir"] += "{}_{}_part/".format(config["graph_name"], world_size)
    device = torch.device("cuda", torch.cuda.current_device())
    set_random_seed(config["random_seed"])
    model, optimizer = create_model_and_optimizer(config, device)
    data = load_data(config)
    TimeRecorder(config["num_layers"], config["num_epochs"], enabled=bool(config.get("record_phases", False)))
    train(model, data, optimizer, config["num_epochs"], config["num_bits"])
    TimeRecorder.ctx.print_total_time()


if __name__ == "__main__":
    main()
