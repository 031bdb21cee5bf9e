"""Forward-only pipeline schedules for inference.

``ScheduleInference.run`` pushes one batch through the stages (receive -> stage forward -> send) and
returns the model output on the last stage; ``ScheduleGeneration`` adds the two-phase API of the
reference (opt_prime/opt_prime/schedule_infer.py:343-454): ``prefill(input_ids, position_ids)`` and
``decode_step(token, position)`` with explicit position ids, returning last-position logits.
"""
from __future__ import annotations

from typing import Any, Dict, Optional

import torch

__all__ = ["ScheduleInference", "ScheduleGeneration"]


class ScheduleInference:
    def __init__(self, engine):
        self.e = engine  # an Optimus_Inference

    @torch.no_grad()
    def run(self, inputs: Optional[Dict[str, Any]]) -> Any:
        e = self.e
        plan, stage = e.plan, e.tpl.stage
        env: Dict[str, Any] = {}
        if e.tpl.is_first_stage():
            if inputs is None:
                raise ValueError("the first stage needs the inputs")
            env.update({k: (e._to_device(v) if isinstance(v, torch.Tensor) else v) for k, v in inputs.items()})
        else:
            e.fwd_in.post_recv(first=True)
            env.update(dict(zip(plan.recv_names(stage), e.fwd_in.wait_recv())))
        args = [env[n] for n in plan.stage_inputs[stage]]
        model_out, outs = e.stage_module(*args)
        env.update(dict(zip(plan.stage_outputs[stage], outs)))
        if not e.tpl.is_last_stage():
            e.fwd_out.send([env[n] for n in plan.send_names(stage)], first=True)
            e.fwd_out.flush()
            return None
        return model_out


class ScheduleGeneration(ScheduleInference):
    def _logits(self, out) -> Optional[torch.Tensor]:
        if out is None:
            return None
        logits = out["logits"] if isinstance(out, dict) else (out[0] if isinstance(out, (tuple, list)) else out)
        return logits[:, -1, :]

    def prefill(self, input_ids: Optional[torch.Tensor], position_ids: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        e = self.e
        inputs = None
        S = None
        if e.tpl.is_first_stage():
            S = input_ids.shape[1]
            if position_ids is None:
                position_ids = torch.arange(S, device=input_ids.device).unsqueeze(0).expand(input_ids.shape[0], S)
            inputs = {"input_ids": input_ids, "position_ids": position_ids}
        S = e._share_int(S)
        out = self.run(inputs)
        e._advance_cache(S)
        return self._logits(out)

    def decode_step(self, token: Optional[torch.Tensor], position: int) -> Optional[torch.Tensor]:
        e = self.e
        inputs = None
        if e.tpl.is_first_stage():
            token = token.view(-1, 1)
            pos = torch.full_like(token, position)
            inputs = {"input_ids": token, "position_ids": pos}
        out = self.run(inputs)
        e._advance_cache(1)
        return self._logits(out)

    def clear_cache(self) -> None:
        self.e.clear_kv_cache()
