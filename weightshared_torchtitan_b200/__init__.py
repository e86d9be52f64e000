"""B200-native shared-W + LoRA linear hot path behind the reference's module API."""
