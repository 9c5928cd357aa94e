from dataclasses import dataclass

import torch


@dataclass
class Transformer2DModelOutput:
    sample: "torch.Tensor" = None

    def __getitem__(self, i):
        return (self.sample,)[i]
