"""Top-k accuracy on integer logits (the reference's ``meters.accuracy``, meters.py:56-70, as its evaluation
loop main.py:150-160 uses it)."""
import torch


def accuracy(output, target, topk=(1,)):
    """Percentage of samples whose label is among the k largest logits, for every k in ``topk``.
    ``output``: [B, classes] (int8 logits or anything comparable; the exponent is irrelevant to the order),
    ``target``: [B] class indices.  Returns a list of 0-dim float tensors like the reference."""
    kmax = max(topk)
    scores = output.to(torch.float32)
    best = scores.topk(kmax, dim=1, largest=True, sorted=True).indices          # [B, kmax]
    hit = best.eq(target.to(best.device).view(-1, 1))                            # [B, kmax]
    n = float(target.shape[0])
    return [hit[:, :k].any(dim=1).float().sum() * (100.0 / n) for k in topk]
