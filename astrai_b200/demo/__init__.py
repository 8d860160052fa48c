"""Small runnable examples: ``python -m astrai_b200.demo.{generate_ar,generate_batch,stream_chat,download}``
(counterparts of the reference's ``scripts/demo/*.py``)."""
