"""Cadence predicates of the training loop.

Steps are counted from 0, and every periodic action (log, checkpoint, evaluation, exit, norm logging) fires
after the ``every``-th completed step: ``(step + 1) % every == 0``, i.e. at steps ``every - 1``,
``2 * every - 1``, ... A checkpoint written at that moment is named for the 0-based step it completes and
a run resumed from it continues at ``step + 1``. The reference uses this form for some actions and
``step > 0 and step % every == 0`` for others (logging and saving one step later, never at step
``every - 1``: ironcore/controller.py:43-70); here one rule serves all of them, so "every N steps" always
means "N optimizer steps have finished since the last time". ``cadence_now`` is the reference's other
predicate, kept for scripts that want its behaviour.
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
    def cadence_now(step: int, every) -> bool:
        return bool(every) and step > 0 and step % every == 0

    _cadence_now = cadence_now

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

    def do_final_checkpoint(self, step=None, last_step=None) -> bool:
        """Whether to save when training ends. Never while profiling or with saving off; with ``step`` (the step
        training ended on) not when the cadence saved that step already; with ``last_step`` (the step the run
        resumed from) as well only when more than one step lies between them, which is the reference's call
        ``do_final_checkpoint(step, last_step)`` (ironcore/controller.py:71-78)."""
        ok = (not self.no_save) and not self.profiling
        if step is not None:
            ok = ok and not self.do_checkpoint(step)
            if last_step is not None:
                ok = ok and step - last_step > 1
        return ok
