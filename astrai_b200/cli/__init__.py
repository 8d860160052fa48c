"""Command-line entry points: ``python -m astrai_b200.cli.{train,serve,generate,preprocess,benchmark}``.

Counterparts of the reference's ``scripts/tools/*.py``; the option names and defaults follow
``docs/guides/params.md`` of the reference so that its launch commands carry over.
"""
