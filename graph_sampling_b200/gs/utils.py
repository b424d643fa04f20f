"""Seed batching helper with the semantics of the reference's SeedGenerator
(python/gs/utils/dataloader.py:4-44)."""
import torch


class SeedGenerator:
    def __init__(self, data: torch.Tensor, batch_size: int, shuffle: bool = False, drop_last: bool = False):
        self.data, self.batch_size, self.shuffle, self.drop_last = data, int(batch_size), shuffle, drop_last

    def __iter__(self):
        if self.shuffle:
            self.data = self.data[torch.randperm(self.data.shape[0], device=self.data.device)]
        self.step = 0
        n = self.data.shape[0]
        self.last_step = n // self.batch_size if self.drop_last else (n + self.batch_size - 1) // self.batch_size
        return self

    def __next__(self):
        if self.step >= self.last_step:
            raise StopIteration
        ret = self.data[self.step * self.batch_size:(self.step + 1) * self.batch_size].clone()
        self.step += 1
        return ret

    def __len__(self):
        return (self.data.shape[0] + self.batch_size - 1) // self.batch_size
