"""Helpers with the names of the reference's `util.utils` (src/util/utils.py)."""
import timeit

import torch


def torch_cuda_identify(print_info=True):
    if torch.cuda.is_available():
        if print_info:
            print(' PyTorch version:', torch.__version__)
            print(' CUDA version \t:', torch.version.cuda)
            print(' GPU cuda:({}) \t: {}'.format(torch.cuda.current_device(), torch.cuda.get_device_name()), '\n', "-" * 50)
        return torch.device('cuda:{}'.format(torch.cuda.current_device()))
    print('cuda is not avaliable !')
    return torch.device('cpu')


def time_stamp_cudasync():
    torch.cuda.synchronize()
    return timeit.default_timer()


def set_dtype(ts: torch.Tensor, dtype: str):
    if dtype == "fp32":
        return ts.float()
    if dtype == "fp16":
        return ts.half()
    raise RuntimeError(f"Unsupported dtype {dtype}")


def transpose_for_scores(x, n_heads, head_size):
    """(B, S, H*W) -> (B, H, S, W) view."""
    return x.view(x.size()[:-1] + (n_heads, head_size)).permute(0, 2, 1, 3)


def seqlen_to_mask(lengths, max_len):
    batch_size = lengths.numel()
    return (torch.arange(0, max_len, device=lengths.device).type_as(lengths).repeat(batch_size, 1).lt(lengths.unsqueeze(1)))
