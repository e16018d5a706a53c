"""Module lookup / replacement by dotted name
(amct_pytorch/utils/model_util.py:19-38)."""


class ModuleHelper:
    def __init__(self, model):
        self.named_module_dict = dict(model.named_modules())

    @staticmethod
    def replace_module_by_name(model, name, mod):
        *parents, leaf = name.split('.')
        owner = model
        for part in parents:
            owner = getattr(owner, part)
        setattr(owner, leaf, mod)
