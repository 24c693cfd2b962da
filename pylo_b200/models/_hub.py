"""Optional Hugging Face Hub mixin.

The reference meta-models inherit ``PyTorchModelHubMixin`` so that
``Model.from_pretrained(hf_key)`` fetches ``config.json`` + safetensors
(pylo/models/Meta_MLP.py:6-11).  When ``huggingface_hub`` is importable the
same mixin is used here, which keeps the checkpoint format identical; when it
is not, ``from_pretrained`` raises with a message that says what is missing
instead of silently building random weights.
"""

try:  # pragma: no cover - depends on the environment
    from huggingface_hub import PyTorchModelHubMixin as HubMixin

    HUB_KW = dict(license="apache-2.0", tags=["learned-optimizer"])
except Exception:  # pragma: no cover

    class HubMixin:  # type: ignore[no-redef]
        def __init_subclass__(cls, **kwargs):
            super().__init_subclass__()

        @classmethod
        def from_pretrained(cls, *args, **kwargs):
            raise RuntimeError(
                f"{cls.__name__}.from_pretrained needs the huggingface_hub package; "
                "pass network=/checkpoint_path= instead"
            )

    HUB_KW = {}
