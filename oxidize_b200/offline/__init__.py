"""Offline checkpoint tools: requantize, prune, merge, LoRA merge (the reference's ``oxidize-quantize``,
``oxidize-prune``, ``oxidize-merge`` crates and the export half of ``oxidize-finetuning``)."""
