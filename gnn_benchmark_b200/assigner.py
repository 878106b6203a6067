"""Assigner: per-node bit widths of the mixed-precision halo exchange, with the reference's class and
method names (self_benchmark/a64fx/assigner.py:7-61).

For every layer and direction ("forward0", "backward1", ...) it keeps one fp32 value per exchanged row:
the bit width (8, 4 or 2) that row is quantised with by `Communicator.comm_with_mixed_quantization`.
With num_bits in {8, 4, 2} the table is constant; with num_bits == -1 the widths are redrawn every
`assign_period` epochs from the three choices with probabilities `assign_weight` (the reference's random
assignment).  The tables live on `device` (default: the current CUDA device), where the quantiser
reads them.
"""
import torch

BIT_CHOICES = (8.0, 4.0, 2.0)


class Assigner(object):
    ctx = None

    def __init__(self, num_bits, num_layers, assign_weight, assign_period, num_send_nodes_on_forward,
                 num_send_nodes_on_backward, device=None):
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        self.num_bits, self.num_layers = num_bits, num_layers
        self.num_send_nodes_on_forward = num_send_nodes_on_forward
        self.num_send_nodes_on_backward = num_send_nodes_on_backward
        self.assign_weight = torch.as_tensor(assign_weight, dtype=torch.float32)
        self.assign_period = assign_period
        fill = float(num_bits) if num_bits != -1 else 0.0
        self.node_dataformat_dict = {}
        for layer in range(num_layers):
            for direction, rows in (("forward", num_send_nodes_on_forward), ("backward", num_send_nodes_on_backward)):
                self.node_dataformat_dict[f"{direction}{layer}"] = torch.full((rows,), fill, dtype=torch.float32,
                                                                              device=device)
        self._choices = torch.tensor(BIT_CHOICES, dtype=torch.float32, device=device)
        Assigner.ctx = self

    def reassign_node_dataformat(self, epoch):
        """Redraw the widths (random mode only) at the start of every assign_period-th epoch."""
        if self.num_bits != -1 or epoch % self.assign_period != 0:
            return
        for table in self.node_dataformat_dict.values():
            if table.numel():
                pick = torch.multinomial(self.assign_weight, table.numel(), replacement=True)
                table.copy_(self._choices[pick.to(table.device)])

    def get_node_dataformat(self, layer):
        return self.node_dataformat_dict[layer]
