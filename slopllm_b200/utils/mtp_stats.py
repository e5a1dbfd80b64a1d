"""Accept-length statistics of speculative decoding (reference: `src/mtp_stats.ts:1-45`)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Sequence


@dataclass
class MtpStats:
    drafts: int                                   # D: drafts per step
    steps: int = 0
    accepted_tokens: int = 0
    histogram: Dict[int, int] = field(default_factory=dict)   # tokens emitted per sequence-step -> count

    def record(self, accepted_per_seq: Sequence[Sequence[int]]) -> None:
        for toks in accepted_per_seq:
            n = len(toks)
            self.steps += 1
            self.accepted_tokens += n
            self.histogram[n] = self.histogram.get(n, 0) + 1

    @property
    def accept_length(self) -> float:
        """Mean tokens emitted per sequence-step (1 = no draft accepted, D + 1 = all)."""
        return self.accepted_tokens / self.steps if self.steps else 0.0

    @property
    def draft_acceptance_rate(self) -> float:
        return (self.accept_length - 1.0) / self.drafts if self.drafts and self.steps else 0.0

    def per_position_rates(self) -> List[float]:
        """P(draft i accepted | reached): from the histogram of emitted counts."""
        rates = []
        for i in range(1, self.drafts + 1):
            reached = sum(c for n, c in self.histogram.items() if n >= i)
            passed = sum(c for n, c in self.histogram.items() if n >= i + 1)
            rates.append(passed / reached if reached else 0.0)
        return rates

    def summary(self) -> dict:
        return {"drafts": self.drafts, "sequence_steps": self.steps, "tokens": self.accepted_tokens,
                "accept_length": round(self.accept_length, 4), "draft_acceptance_rate": round(self.draft_acceptance_rate, 4),
                "per_position": [round(r, 4) for r in self.per_position_rates()],
                "histogram": {str(k): v for k, v in sorted(self.histogram.items())}}
