from .passes import BaseModuleFusionPass, InsertQuantizeModulePass, ModelOptimizer, ReplaceNpuQuantModulePass

__all__ = ['BaseModuleFusionPass', 'InsertQuantizeModulePass', 'ModelOptimizer', 'ReplaceNpuQuantModulePass']
