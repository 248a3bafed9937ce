from emmy.compiler.ir.stmt.base import Stmt
from emmy.compiler.ir.stmt.blocks import Cond, Loop, StridedLoop
from emmy.compiler.ir.stmt.body import Body
from emmy.compiler.ir.stmt.leaves import Accum, Assign, Init, Let, Load, Select, SelectBranch, Write

__all__ = ['Accum', 'Assign', 'Body', 'Cond', 'Init', 'Let', 'Load', 'Loop', 'Select', 'SelectBranch', 'Stmt', 'StridedLoop', 'Write']
