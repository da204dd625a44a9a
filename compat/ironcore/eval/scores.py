"""Score helpers: the reference ships this module path without content (ironcore/eval/scores.py is a licence header
only); task scores are computed inside each task's ``process`` (``ironcore.eval.tasks``)."""
