import torch


def segment_csr(src, indptr, out=None, reduce="sum"):
    lengths = torch.diff(indptr)
    return torch.segment_reduce(src, reduce, lengths=lengths, axis=0, unsafe=True)
