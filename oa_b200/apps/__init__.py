"""Command-line tools: `python -m oa_b200.apps.modelctl` and `python -m oa_b200.apps.datasetctl`."""
