"""Views that relate the chunk-layout tensors of the CUDA library to the stage outputs of oracle/kernel_plan.py."""
import torch


def image_to_matrix(img, rows, cols, SI, SJ):
    """Decode a plain operand image (bf16 tensor, flat) into a (rows, cols) matrix."""
    i = torch.arange(rows)[:, None]
    j = torch.arange(cols)[None, :]
    off = (i // 8) * SI + (j // 8) * SJ + (i % 8) * 16 + (j % 8) * 2
    return img.reshape(-1)[(off // 2).reshape(-1)].reshape(rows, cols)


def decode_items(t, fn):
    """Apply fn to every (b, n, h) item of a chunk-layout tensor -> stacked (B*H, NC, ...) like the plan's tensors."""
    B, NC, H = t.shape[:3]
    out = []
    for b in range(B):
        for h in range(H):
            out.append(torch.stack([fn(t[b, n, h]) for n in range(NC)]))
    return torch.stack(out)


def state_to_matrix(hs):
    """(E,16,128,8) saved state -> (E, 128 d, 128 v)."""
    E = hs.shape[0]
    return hs.permute(0, 2, 1, 3).reshape(E, 128, 128)
