"""Transition detector against a line-by-line replay of the reference driver's state machine
(main_conv_ff.py:211-242)."""
import torch

from spion_b200.transition import TransitionDetector


def reference_replay(seq, num_layers):
    """The driver's variables and branches, kept in the driver's order."""
    before_attn, current_attn, before_distance, current_distance, diff = [], [], [], [], []
    transition, at = False, None
    for step, attn_lst in enumerate(seq):
        if transition:
            break
        if len(before_attn) == 0:
            for l in range(num_layers):
                before_attn.append(attn_lst[l]); current_attn.append(attn_lst[l])
        else:
            for l in range(num_layers):
                current_attn[l] = attn_lst[l]
            if len(before_distance) == 0:
                for l in range(num_layers):
                    d = torch.sqrt(torch.sum(torch.pow(before_attn[l] - current_attn[l], 2)))
                    before_distance.append(d); current_distance.append(d); diff.append(0)
            else:
                cnt = 0
                for l in range(num_layers):
                    current_distance[l] = torch.sqrt(torch.sum(torch.pow(before_attn[l] - current_attn[l], 2)))
                    diff[l] = (abs(current_distance[l] - before_distance[l]) / before_distance[l]) * 100
                    before_distance[l] = current_distance[l]
                    if int(diff[l]) < 15:
                        cnt += 1
                if cnt == num_layers:
                    transition, at = True, step + 1
                else:
                    for l in range(num_layers):
                        before_attn[l] = current_attn[l]
    return transition, at


def make_seq(kind, n=8, L=16, layers=2):
    g = torch.Generator().manual_seed(7)
    base = [torch.softmax(torch.randn(L, L, generator=g), -1) for _ in range(layers)]
    seq = []
    for k in range(n):
        if kind == "settling":
            amp = 0.5 * (0.9 ** k) if k < 4 else 0.5 * (0.9 ** 4)
        elif kind == "noisy":
            amp = 0.5 * (2.0 if k % 2 else 0.3)
        else:
            amp = 0.5 / (k + 1)
        seq.append([b + amp * torch.randn(L, L, generator=g) for b in base])
    return seq


def test_matches_driver_replay():
    for kind in ("settling", "noisy", "decay"):
        seq = make_seq(kind)
        det = TransitionDetector(2)
        fired = None
        for k, maps in enumerate(seq):
            if det.update(maps) and fired is None:
                fired = k + 1
        want, at = reference_replay(seq, 2)
        assert det.transition == want and fired == at, kind


def test_needs_three_checks_and_latches():
    maps = [torch.eye(4), torch.eye(4)]
    det = TransitionDetector(2)
    assert det.update(maps) is False
    assert det.update([m + 0.1 for m in maps]) is False
    assert det.update([m + 0.2 for m in maps]) is False     # distance doubled: 100 % change, keep training dense
    assert det.update([m + 0.41 for m in maps]) is True      # distance 0.8 -> 0.84 against the refreshed map: 5 % < 15 %
    assert det.update(maps) is True                          # latched
