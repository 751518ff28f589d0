from .mask_sigmoid import *
from .mask_softmax import *
