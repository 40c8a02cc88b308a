"""Built artefacts (kernel library, native host module) land here; see pie_b200._build."""
