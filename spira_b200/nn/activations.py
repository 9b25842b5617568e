"""Feature-wise activations on SparseTensors (reference: spira/nn/activations.py:8-18)."""
__all__ = ['ReLU', 'ReLU6', 'LeakyReLU']

import torch

from spira_b200.utils.apply import fapply


class ReLU(torch.nn.ReLU):
    def forward(self, input):
        return fapply(input, super().forward)


class ReLU6(torch.nn.ReLU6):
    def forward(self, input):
        return fapply(input, super().forward)


class LeakyReLU(torch.nn.LeakyReLU):
    def forward(self, input):
        return fapply(input, super().forward)
