__all__ = ['ScalarOrIterable', 'ScalarOrTuple']

from typing import Iterable, Tuple, TypeVar, Union

T = TypeVar('T')
ScalarOrTuple = Union[T, Tuple[T, ...]]
ScalarOrIterable = Union[T, Iterable[T]]
