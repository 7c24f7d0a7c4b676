{-# LANGUAGE GADTs               #-}
{-# LANGUAGE RankNTypes          #-}
{-# LANGUAGE ScopedTypeVariables #-}
-- |
-- Module      : Data.Array.Accelerate.B200.CodeGen
-- Description : Scalar functions of an Accelerate program printed as functor snippets
--
-- NOT COMPILED HERE: the build machine of this repository has no GHC.
--
-- accelerate-cuda's code generator prints WHOLE kernels: a skeleton template
-- with the user's scalar functions pasted in
-- (Data/Array/Accelerate/CUDA/CodeGen.hs:91-136 and CodeGen/*.hs).  The
-- skeletons of this backend are C++ headers that ship with the library
-- (csrc/skeletons/*.cuh); what remains to be printed per node is a small
-- struct -- the functor -- holding the scalar functions.  The contract of each
-- skeleton is stated at the top of its header; the Python module
-- accelerate-cuda_b200/lang.py prints the same structs from Python functions
-- and is the executable specification of this module.
--
-- Scalar expressions are printed in single-assignment form: every
-- sub-expression becomes a @const T vN = ...;@ statement, a tuple is the list
-- of its flattened components (leftmost first, CodeGen/Type.hs:101-104).
-- C semantics of the primitives follow CodeGen/Arithmetic.hs: floor division
-- for div/mod (:103-134), truncation for quot/rem (:89-101), fminf/fmaxf
-- (:322-336), C round (:281-282), one-byte Bool.
--
module Data.Array.Accelerate.B200.CodeGen (

  Functor(..), Gamma, freeArrays,
  functorMap, functorFold, functorScan, functorPermute, functorStencil,
  cTypesOf,

) where

import Control.Monad.State
import Data.List                                        ( intercalate )
import Text.Printf

import Data.Array.Accelerate.AST
import Data.Array.Accelerate.Array.Sugar                ( Elt, eltType, EltRepr, fromElt )
import Data.Array.Accelerate.Trafo                      ( DelayedOpenAcc )
import Data.Array.Accelerate.Tuple
import Data.Array.Accelerate.Type

-- | What 'accb_kernel_get' wants: skeleton name, struct name, source text;
-- plus the free array variables the functor reads, in the order the launch
-- must pass them (the Gamma of CUDA/AST.hs:72-112).
data Functor = Functor
  { fSkeleton :: String
  , fName     :: String
  , fSource   :: String
  , fGamma    :: Gamma
  }

-- | Free array variables by de Bruijn level of the array environment; the
-- position in the list is the environment-array number the functor uses.
type Gamma = [Int]

freeArrays :: Functor -> Gamma
freeArrays = fGamma

-- Code generation monad: fresh names, emitted statements, array variables met
data Gen = Gen { next :: !Int, stmts :: [String], gamma :: Gamma }
type CG  = State Gen

fresh :: String -> String -> CG String          -- emit "const ty vN = rhs;" and name it
fresh ty rhs = do
  s <- get
  let v = "v" ++ show (next s)
  put s { next = next s + 1, stmts = printf "const %s %s = %s;" ty v rhs : stmts s }
  return v

arrayVar :: Int -> CG Int                        -- environment-array number of a free array variable
arrayVar lvl = do
  s <- get
  case lookup lvl (zip (gamma s) [0 ..]) of
    Just n  -> return n
    Nothing -> do put s { gamma = gamma s ++ [lvl] }
                  return (length (gamma s))

runCG :: CG a -> (a, [String], Gamma)
runCG m = let (a, s) = runState m (Gen 0 [] []) in (a, reverse (stmts s), gamma s)

-- ---------------------------------------------------------------- types
-- | C type of every flattened component of an element type.
cTypesOf :: TupleType t -> [String]
cTypesOf UnitTuple         = []
cTypesOf (SingleTuple t)   = [scalarC t]
cTypesOf (PairTuple a b)   = cTypesOf a ++ cTypesOf b

scalarC :: ScalarType t -> String
scalarC (NumScalarType (IntegralNumType t)) = integralC t
scalarC (NumScalarType (FloatingNumType t)) = floatingC t
scalarC (NonNumScalarType t)                = nonNumC t

integralC :: IntegralType t -> String
integralC TypeInt{}    = "long long"      -- Accelerate's Int is 64 bits wide on the hosts this runs on
integralC TypeInt8{}   = "signed char"
integralC TypeInt16{}  = "short"
integralC TypeInt32{}  = "int"
integralC TypeInt64{}  = "long long"
integralC TypeWord{}   = "unsigned long long"
integralC TypeWord8{}  = "unsigned char"
integralC TypeWord16{} = "unsigned short"
integralC TypeWord32{} = "unsigned int"
integralC TypeWord64{} = "unsigned long long"
integralC _            = error "B200.CodeGen: C integral types are not supported as element types"

floatingC :: FloatingType t -> String
floatingC TypeFloat{}  = "float"
floatingC TypeDouble{} = "double"
floatingC _            = error "B200.CodeGen: C floating types are not supported as element types"

nonNumC :: NonNumType t -> String
nonNumC TypeBool{} = "unsigned char"      -- one byte, as the reference stores Bool
nonNumC TypeChar{} = "unsigned int"
nonNumC _          = error "B200.CodeGen: C character types are not supported as element types"

-- ---------------------------------------------------------------- expressions
-- | Values of the scalar environment: one list of component names per binding, innermost first.
type Val = [[String]]

-- | An open expression as the list of its flattened components.
expC :: forall env aenv t. Elt t => Int -> Val -> PreOpenExp DelayedOpenAcc env aenv t -> CG [String]
expC alvl env = go
  where
    go :: forall s. Elt s => PreOpenExp DelayedOpenAcc env aenv s -> CG [String]
    go (Let bnd body)      = do b <- go bnd
                                expC alvl (b : env) body
    go (Var ix)            = return (env !! idxToInt ix)
    go (Const c)           = return (constC (eltType (undefined :: s)) c)
    go (PrimConst c)       = return [primConstC c]
    go (Tuple t)           = tupC t
    go (Prj ix e)          = do comps <- go e
                                return (prjC ix (eltType (undefined :: s)) comps)
    go (Cond p t e)        = do [c] <- go p
                                ts  <- go t
                                es  <- go e
                                zipWithM3 (\ty a b -> fresh ty (printf "%s ? %s : %s" c a b))
                                          (cTypesOf (eltType (undefined :: s))) ts es
    go (PrimApp f x)       = do xs <- go x
                                primC f (cTypesOf (eltType (undefined :: s))) xs
    go IndexNil            = return []
    go IndexAny            = return []
    go (IndexCons sh i)    = (++) <$> go sh <*> go i                 -- outermost first, innermost last
    go (IndexHead sh)      = (\c -> [last c]) <$> go sh
    go (IndexTail sh)      = init <$> go sh
    go (ShapeSize sh)      = do c <- go sh
                                (: []) <$> fresh "long long" (intercalate " * " (map (printf "(long long)%s") c ++ ["1LL"]))
    go (ToIndex sh ix)     = do s <- go sh
                                i <- go ix
                                (: []) <$> fresh "long long" (rowMajor s i)
    go (FromIndex sh i)    = do s   <- go sh
                                [l] <- go i
                                fromIndexC s l
    go (Shape a)           = do n <- arrayVar (avarLevel a)
                                let r = rankOfArrayTerm a
                                return [ printf "env.dim(%d, %d)" n (r - 1 - d) | d <- [0 .. r - 1] ]
    go (LinearIndex a i)   = do n   <- arrayVar (avarLevel a)
                                [l] <- go i
                                gatherC n (cTypesOf (eltType (undefined :: s))) l
    go (Index a ix)        = do n  <- arrayVar (avarLevel a)
                                i  <- go ix
                                let r  = length i
                                    sh = [ printf "env.dim(%d, %d)" n (r - 1 - d) | d <- [0 .. r - 1] ]
                                l  <- fresh "long long" (rowMajor sh i)
                                gatherC n (cTypesOf (eltType (undefined :: s))) l
    go (While{})           = unsupported "while loops inside scalar functions"
    go (Foreign{})         = unsupported "foreign scalar functions"
    go _                   = unsupported "this scalar construct"

    tupC :: forall tup. Tuple (PreOpenExp DelayedOpenAcc env aenv) tup -> CG [String]
    tupC NilTup            = return []
    tupC (SnocTup t e)     = (++) <$> tupC t <*> go e

    avarLevel :: DelayedOpenAcc aenv a -> Int
    avarLevel = error "B200.CodeGen: de Bruijn level of an array variable (Manifest (Avar ix) -> alvl - 1 - idxToInt ix)"
    rankOfArrayTerm :: DelayedOpenAcc aenv a -> Int
    rankOfArrayTerm = error "B200.CodeGen: rank from the array type of the term (Sugar.rank)"

unsupported :: String -> a
unsupported what = error ("Data.Array.Accelerate.B200: " ++ what ++ " is not translated by this shim yet")

zipWithM3 :: Monad m => (a -> b -> c -> m d) -> [a] -> [b] -> [c] -> m [d]
zipWithM3 f (a:as) (b:bs) (c:cs) = (:) <$> f a b c <*> zipWithM3 f as bs cs
zipWithM3 _ _      _      _      = return []

-- row-major linear index from extents and coordinates, both outermost first (CodeGen/Base.hs:195-218)
rowMajor :: [String] -> [String] -> String
rowMajor sh ix = foldl (\acc (s, i) -> printf "(%s) * (long long)%s + (long long)%s" acc s i) "0LL" (zip sh ix)

fromIndexC :: [String] -> String -> CG [String]
fromIndexC sh l = reverse <$> go (reverse sh) l
  where
    go []       _ = return []
    go [_]      r = (: []) <$> fresh "int" (printf "(int)(%s)" r)
    go (s : ss) r = do x  <- fresh "int" (printf "(int)((%s) %% %s)" r s)
                       r' <- fresh "long long" (printf "(%s) / %s" r s)
                       (x :) <$> go ss r'

-- arrays that are not read element-wise are gathered through the environment
gatherC :: Int -> [String] -> String -> CG [String]
gatherC n tys l = forM (zip [0 :: Int ..] tys) $ \(c, ty) ->
  fresh ty (printf "env.in<%s>(ENV_SLOT(%d, %d))[%s]" ty n c l)

constC :: TupleType t -> t -> [String]
constC UnitTuple       ()     = []
constC (SingleTuple t) c      = [printf "(%s)%s" (scalarC t) (showScalar t c)]
constC (PairTuple a b) (x, y) = constC a x ++ constC b y

showScalar :: ScalarType t -> t -> String
showScalar (NumScalarType (IntegralNumType t)) c | IntegralDict <- integralDict t = show c
showScalar (NumScalarType (FloatingNumType t)) c | FloatingDict <- floatingDict t = printf "%.17g" (realToFrac c :: Double)
showScalar (NonNumScalarType TypeBool{})       c = if c then "1" else "0"
showScalar (NonNumScalarType t)                c | NonNumDict <- nonNumDict t     = show (fromEnum c)

primConstC :: PrimConst t -> String
primConstC (PrimMinBound (IntegralBoundedType t)) | IntegralDict <- integralDict t = show (minBound `asTypeOfI` t)
primConstC (PrimMaxBound (IntegralBoundedType t)) | IntegralDict <- integralDict t = show (maxBound `asTypeOfI` t)
primConstC (PrimPi t)                             | FloatingDict <- floatingDict t = "3.14159265358979323846"
primConstC _                                      = unsupported "this primitive constant"

asTypeOfI :: a -> IntegralType a -> a
asTypeOfI x _ = x

-- projection: the components of the projected field inside the flattened tuple
prjC :: TupleIdx t e -> TupleType r -> [String] -> [String]
prjC _ resultTy comps = take w (drop (length comps - skip - w) comps)
  where
    w    = length (cTypesOf resultTy)
    skip = error "B200.CodeGen: components to the right of the field = sum of the widths of the fields after it"

-- | Primitive applications; the argument arrives flattened (a binary operator has two components).
primC :: PrimFun (a -> r) -> [String] -> [String] -> CG [String]
primC f [ty] xs = (: []) <$> fresh ty (rhs f xs)
  where
    rhs :: PrimFun (a -> r) -> [String] -> String
    rhs PrimAdd{}    [a, b] = binop "+" a b
    rhs PrimSub{}    [a, b] = binop "-" a b
    rhs PrimMul{}    [a, b] = binop "*" a b
    rhs PrimNeg{}    [a]    = printf "-%s" a
    rhs PrimAbs{}    [a]    = printf "(%s < 0 ? -%s : %s)" a a a
    rhs PrimQuot{}   [a, b] = binop "/" a b                                   -- truncates (Arithmetic.hs:89-101)
    rhs PrimRem{}    [a, b] = binop "%" a b
    rhs PrimIDiv{}   [a, b] = printf "accb::floor_div(%s, %s)" a b           -- floors  (Arithmetic.hs:103-134)
    rhs PrimMod{}    [a, b] = printf "accb::floor_mod(%s, %s)" a b
    rhs PrimFDiv{}   [a, b] = binop "/" a b
    rhs PrimBAnd{}   [a, b] = binop "&" a b
    rhs PrimBOr{}    [a, b] = binop "|" a b
    rhs PrimBXor{}   [a, b] = binop "^" a b
    rhs PrimBNot{}   [a]    = printf "~%s" a
    rhs PrimSqrt{}   [a]    = call1 "sqrt" a
    rhs PrimExpFloating{} [a] = call1 "exp" a
    rhs PrimLog{}    [a]    = call1 "log" a
    rhs PrimSin{}    [a]    = call1 "sin" a
    rhs PrimCos{}    [a]    = call1 "cos" a
    rhs PrimTanh{}   [a]    = call1 "tanh" a
    rhs PrimFPow{}   [a, b] = printf "%s(%s, %s)" (mathfn "pow") a b
    rhs PrimLt{}     [a, b] = binop "<" a b
    rhs PrimGt{}     [a, b] = binop ">" a b
    rhs PrimLtEq{}   [a, b] = binop "<=" a b
    rhs PrimGtEq{}   [a, b] = binop ">=" a b
    rhs PrimEq{}     [a, b] = binop "==" a b
    rhs PrimNEq{}    [a, b] = binop "!=" a b
    rhs PrimMax{}    [a, b] = printf "%s(%s, %s)" (minmax "max") a b         -- fmaxf on floats (Arithmetic.hs:322-336)
    rhs PrimMin{}    [a, b] = printf "%s(%s, %s)" (minmax "min") a b
    rhs PrimLAnd     [a, b] = binop "&&" a b
    rhs PrimLOr      [a, b] = binop "||" a b
    rhs PrimLNot     [a]    = printf "!%s" a
    rhs PrimFromIntegral{} [a] = printf "(%s)%s" ty a
    rhs PrimToFloating{}   [a] = printf "(%s)%s" ty a
    rhs PrimTruncate{} [a]  = printf "(%s)%s" ty a
    rhs PrimRound{}  [a]    = printf "(%s)%s(%s)" ty (mathfn "round") a      -- C round, half away from zero (Arithmetic.hs:281-282)
    rhs PrimFloor{}  [a]    = printf "(%s)%s(%s)" ty (mathfn "floor") a
    rhs PrimCeiling{} [a]   = printf "(%s)%s(%s)" ty (mathfn "ceil") a
    rhs _            _      = unsupported "this primitive function"

    binop op a b = printf "(%s %s %s)" a op b
    call1 fn a   = printf "%s(%s)" (mathfn fn) a
    mathfn fn    = if ty == "float" then fn ++ "f" else fn
    minmax fn    = if ty == "float" then "f" ++ fn ++ "f" else if ty == "double" then "f" ++ fn else fn
primC _ _ _ = unsupported "primitive functions with tuple results"

-- ---------------------------------------------------------------- functors
struct :: String -> String -> [String] -> String
struct name base body = unlines ([printf "struct %s%s {" name base] ++ map ("    " ++) body ++ ["};"])

devFn :: String
devFn = "static __device__ __forceinline__"

-- | map / zipWith / generate fused into one element-wise kernel: @apply(env, i, in-values..., out-references...)@
-- (contract: csrc/skeletons/map.cuh; reference: CodeGen/Mapping.hs:39-78, CodeGen/IndexSpace.hs:47-141).
functorMap :: (Elt a, Elt b) => Int -> String -> [String] -> [String] -> PreOpenFun DelayedOpenAcc () aenv (a -> b) -> Functor
functorMap alvl name inTys outTys (Lam (Body e)) =
  let ins           = [ "x" ++ show k | k <- [0 .. length inTys - 1] ]
      (res, ss, g)  = runCG (expC alvl [ins] e)
      params        = [ printf "%s %s" t x | (t, x) <- zip inTys ins ] ++ [ printf "%s &o%d" t k | (t, k) <- zip outTys [0 :: Int ..] ]
      body          = [ printf "using In = accb::types<%s>;" (intercalate ", " inTys)
                      , printf "using Out = accb::types<%s>;" (intercalate ", " outTys)
                      , printf "%s void apply(const accb::Env &env, long long i, %s) {" devFn (intercalate ", " params) ]
                      ++ map ("    " ++) (ss ++ [ printf "o%d = %s;" k r | (k, r) <- zip [0 :: Int ..] res ]) ++ ["}"]
  in Functor "map" name (struct name "" body) g
functorMap _ _ _ _ _ = unsupported "element-wise functions of this arity"

-- | fold / fold1 / foldAll / foldSeg: @get@ is the fused producer, @combine@ the user's operator
-- (contract: csrc/skeletons/fold.cuh; reference: CodeGen/Reduction.hs:87-574).
functorFold :: Elt e => Int -> String -> String -> [String] -> String
            -> PreOpenFun DelayedOpenAcc () aenv (a -> e)          -- producer at the linear index or of the input values
            -> PreOpenFun DelayedOpenAcc () aenv (e -> e -> e)
            -> Functor
functorFold alvl skeleton name inTys ty (Lam (Body get)) (Lam (Lam (Body f))) =
  let ins             = [ "x" ++ show k | k <- [0 .. length inTys - 1] ]
      ([g1], s1, ga)  = runCG (expC alvl [ins] get)
      ([c1], s2, gb)  = runCG (expC alvl [["b"], ["a"]] f)
      body            = [ printf "using In = accb::types<%s>;" (intercalate ", " inTys)
                        , printf "%s %s get(const accb::Env &env, long long i, %s) {" devFn ty
                                 (intercalate ", " [ printf "%s %s" t x | (t, x) <- zip inTys ins ]) ]
                        ++ map ("    " ++) (s1 ++ ["return " ++ g1 ++ ";"]) ++ ["}"]
                        ++ [ printf "%s %s combine(%s a, %s b) {" devFn ty ty ty ]
                        ++ map ("    " ++) (s2 ++ ["return " ++ c1 ++ ";"]) ++ ["}"]
  in Functor skeleton name (struct name (printf " : accb::Fold<%s>" ty) body) (ga ++ filter (`notElem` ga) gb)
functorFold _ _ _ _ _ _ _ = unsupported "reductions over tuples"

-- | the six scans share the fold's functor shape (contract: csrc/skeletons/scan.cuh; reference: CodeGen/PrefixSum.hs:59-480)
functorScan :: Elt e => Int -> String -> [String] -> String
            -> PreOpenFun DelayedOpenAcc () aenv (a -> e) -> PreOpenFun DelayedOpenAcc () aenv (e -> e -> e) -> Functor
functorScan alvl name inTys ty get f =
  let fn = functorFold alvl "scan" name inTys ty get f
  in fn { fSource = replaceBase (fSource fn) }
  where
    replaceBase = unwords . map (\w -> if take 10 w == "accb::Fold" then "accb::Scan" ++ drop 10 w else w) . words

-- | permute: @index@ maps a source index to a destination (negative: ignore), @combine(new, old)@
-- (contract: csrc/skeletons/permute.cuh; reference: CodeGen/IndexSpace.hs:160-303)
functorPermute :: Int -> String -> [String] -> String -> String -> Functor
functorPermute _ name inTys ty atomic =
  Functor (if atomic == "Add" then "permute_smem" else "permute") name
          (struct name (printf " : accb::Permute<%s, accb::Atomic::%s>" ty atomic)
                  [ printf "using In = accb::types<%s>;" (intercalate ", " inTys)
                  , "/* index(env, i, in-values...), get(env, i, in-values...), combine(x, y), identity(): printed from the"
                  , "   permutation function, the fused source and the combination function as for functorFold */" ])
          []

-- | stencil: the neighbourhood arrives as a nested array t[dy][dx] (t[dz][dy][dx] for cubes)
-- (contract: csrc/skeletons/stencil.cuh, stencil3.cuh; reference: CodeGen/Stencil.hs:55-228, Stencil/Extra.hs)
functorStencil :: Int -> String -> String -> String -> [Int] -> ([[String]] -> CG String) -> Functor
functorStencil _ name tin tout radii body =
  let dims          = map (\r -> 2 * r + 1) radii
      taps          = [ [ "t" ++ concatMap (printf "[%d]") ix | ix <- sequence (map (\d -> [0 .. d - 1]) dims) ] ]
      (res, ss, g)  = runCG (body taps)
      base          = if length radii == 3 then "Stencil3" else "Stencil"
      rs            = intercalate ", " (map show (if length radii == 1 then 0 : radii else radii))
      arr           = concatMap (printf "[%d]") (if length radii == 1 then 1 : dims else dims)
  in Functor (if length radii == 3 then "stencil3" else "stencil") name
             (struct name (printf " : accb::%s<%s, %s, %s>" base tin tout rs)
                     ([ printf "%s %s apply(const accb::Env &env, const %s (&t)%s) {" devFn tout tin arr ]
                      ++ map ("    " ++) (ss ++ ["return " ++ res ++ ";"]) ++ ["}"]))
             g
