"""Seed batching helper with the semantics of the reference's SeedGenerator
(python/gs/utils/dataloader.py:4-44) and the block builders of python/gs/utils/to_dgl_block.py:5-25."""
import torch


def create_block_from_csc(indptr, indices, e_ids, num_src, num_dst):
    """Message-flow block over a relabelled CSC sample.  With DGL importable this is the reference's
    DGLBlock (python/gs/utils/to_dgl_block.py:5-17); without it, the same fields as a plain `Block`."""
    try:
        import dgl
        from dgl.heterograph import DGLBlock
    except ImportError:
        from .matrix import Block
        return Block("csc", indptr, indices, int(num_src), int(num_dst), None, e_ids, None)
    hgidx = dgl.heterograph_index.create_unitgraph_from_csr(
        2, num_src, num_dst, indptr, indices, e_ids, formats=["coo", "csr", "csc"], transpose=True)
    return DGLBlock(hgidx, (["_N"], ["_N"]), ["_E"])


def create_block_from_coo(row, col, num_src, num_dst):
    """As `create_block_from_csc` for a relabelled COO sample (python/gs/utils/to_dgl_block.py:20-25)."""
    try:
        import dgl
        from dgl.heterograph import DGLBlock
    except ImportError:
        from .matrix import Block
        return Block("coo", row, col, int(num_src), int(num_dst), None, None, None)
    hgidx = dgl.heterograph_index.create_unitgraph_from_coo(
        2, num_src, num_dst, row, col, formats=["coo", "csr", "csc"])
    return DGLBlock(hgidx, (["_N"], ["_N"]), ["_E"])


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
