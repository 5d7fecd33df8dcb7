"""Helpers with the names of the reference's `util.utils` (src/util/utils.py)."""
import re
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


def transpose_for_scores1(x):
    """`transpose_for_scores` with the reference's fixed 12 heads of 64 (src/util/utils.py:36-39)."""
    return transpose_for_scores(x, 12, 64)


_TUNING_LINE = re.compile(r"num_warp(\d+)\s*\|\s*m(\d+)n(\d+)\s*\|\s*bs:(\d+)\s*\|\s*seq:(\d+)\s*\|\s*([\d.]+)\s*ms/iter\s*\|\s*Speedup/FA2:\s*([\d.]+)")


def read_config_file(file_path):
    """Parses a tuning log of the reference's attention benchmark (lines `num_warpW | mMnN | bs:B | seq:S | T ms/iter |
    Speedup/FA2: X`) into {batch: {seq_len: [(BLOCK_M, BLOCK_N, num_warps), ...]}} in file order (src/util/utils.py:50-69)."""
    table = {}
    with open(file_path, "r") as fh:
        for line in fh:
            m = _TUNING_LINE.match(line)
            if m is None:
                continue
            warps, bm, bn, bs, seq = (int(m.group(i)) for i in range(1, 6))
            table.setdefault(bs, {}).setdefault(seq, []).append((bm, bn, warps))
    return table


def get_best_config(config_data, batch_size, seq_len):
    """First (BLOCK_M, BLOCK_N, num_warps) logged for this batch size and sequence length (src/util/utils.py:72-77)."""
    try:
        return config_data[batch_size][seq_len][0]
    except (KeyError, IndexError):
        raise ValueError(f"no tuned configuration for batch {batch_size}, seq_len {seq_len}")

