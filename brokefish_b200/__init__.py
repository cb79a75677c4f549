"""brokefish_b200: the Brokefish network evaluator rebuilt for NVIDIA B200 (sm_100a).

Public surface (same names as the reference's ``brokefish.nn`` and
``brokefish.search.make_evaluator``):

* :func:`brokefish_b200.nn.encoder_impl` -> :class:`FusedEncoder`
* :class:`brokefish_b200.nn.model.BrokefishNet`
* :func:`brokefish_b200.evaluator.make_evaluator`
* :class:`brokefish_b200.evaluator.ShardedEvaluator` (positions split across GPUs)
"""

__version__ = "0.1"
