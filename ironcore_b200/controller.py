"""Cadence predicates of the training loop.
``now``  : step > 0 and step % every == 0      ``next`` : (step + 1) % every == 0
(Behavioural reference: ironcore/controller.py:12-78.)"""

from __future__ import annotations


class TrainingControl:
    def __init__(self, config):
        self.config = config
        t, o = config.trainer, config.operation
        self.log_interval = t.log_interval
        self.save_interval = t.save_checkpoint_steps
        self.eval_interval = o.eval_interval
        self.train_steps = o.train_steps
        self.exit_interval = o.exit_interval
        self.no_save = o.no_save or not t.model_path
        self.profiling = config.utils.profile_torch or config.utils.profile_nsys

    @staticmethod
    def _cadence_now(step: int, every) -> bool:
        return bool(every) and step > 0 and step % every == 0

    @staticmethod
    def _cadence_next(step: int, every) -> bool:
        return bool(every) and (step + 1) % every == 0

    def do_log(self, step: int) -> bool:
        return self._cadence_next(step, self.log_interval)

    def do_checkpoint(self, step: int) -> bool:
        return (not self.no_save) and self._cadence_next(step, self.save_interval)

    def do_eval(self, step: int) -> bool:
        return self.config.trainer.do_eval and self._cadence_next(step, self.eval_interval)

    def do_eval_subtask(self, step: int) -> bool:
        return self.config.trainer.do_eval_subtask and self._cadence_next(step, self.eval_interval)

    def do_exit(self, step: int) -> bool:
        return self.exit_interval is not None and self._cadence_next(step, self.exit_interval)

    def _norm_cadence(self, mode, step):
        if mode == "log":
            return self.do_log(step)
        if mode == "checkpoint":
            return self._cadence_next(step, self.save_interval)
        return False

    def do_grad_norm(self, step: int) -> bool:
        return self._norm_cadence(self.config.trainer.grad_norm_log_interval, step)

    def do_param_norm(self, step: int) -> bool:
        return self._norm_cadence(self.config.trainer.param_norm_log_interval, step)

    def do_final_checkpoint(self) -> bool:
        return (not self.no_save) and not self.profiling
