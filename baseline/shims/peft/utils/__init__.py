"""``peft.utils`` names the reference imports; all raise when called (see the package docstring)."""


def _missing(*args, **kwargs):
    raise NotImplementedError('peft is not installed; this shim only satisfies imports')


load_peft_weights = get_peft_model_state_dict = set_peft_model_state_dict = _missing
