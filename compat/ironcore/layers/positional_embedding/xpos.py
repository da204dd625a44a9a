"""xPos positional embedding: the reference ships this module path without an implementation
(ironcore/layers/positional_embedding/xpos.py is a licence header only); it is kept importable here for the same
reason and defines nothing."""
