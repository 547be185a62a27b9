"""Dense -> sparse transition detector of the reference driver (main_conv_ff.py:211-242).

Every ``eval_frequency`` steps the driver compares each layer's mean attention map with the one
from the previous check: d_l = ||A_prev - A_cur||_F (``frobenius_distance``, :25-32).  From the
third check on it looks at the relative change of that distance,
``diff_l = |d_cur - d_prev| / d_prev * 100``, and switches to the sparse phase once
``int(diff_l) < 15`` holds for every layer.  State is carried exactly as the driver does:
``before_attn`` is refreshed only while no transition has been declared.
"""
from __future__ import annotations

import torch


class TransitionDetector:
    def __init__(self, num_layers: int, percent: float = 15.0):
        self.num_layers = num_layers
        self.percent = percent
        self.before_attn = []
        self.before_distance = []
        self.diff = [0.0] * num_layers
        self.transition = False
        self.transition_check = None
        self.checks = 0

    @staticmethod
    def frobenius_distance(A: torch.Tensor, B: torch.Tensor) -> torch.Tensor:
        return torch.sqrt(torch.sum(torch.pow(A - B, 2)))

    def update(self, attn_lst) -> bool:
        """Feed the per-layer [L, L] maps of one check; returns True once the switch is due."""
        if self.transition:
            return True
        self.checks += 1
        cur = [a.detach() for a in attn_lst]
        if not self.before_attn:                                   # first check: remember the maps (:213-216)
            self.before_attn = cur
            return False
        dist = [float(self.frobenius_distance(b, c)) for b, c in zip(self.before_attn, cur)]
        if not self.before_distance:                               # second check: first distances (:221-225)
            self.before_distance = dist
            return False
        ok = 0
        for l in range(self.num_layers):                           # later checks (:227-236)
            self.diff[l] = abs(dist[l] - self.before_distance[l]) / self.before_distance[l] * 100
            self.before_distance[l] = dist[l]
            if int(self.diff[l]) < self.percent:
                ok += 1
        if ok == self.num_layers:
            self.transition = True
            self.transition_check = self.checks
        else:
            self.before_attn = cur                                 # (:241-242)
        return self.transition
